// Entry points nk_broadcast, nk_binary, nk_fill_fun, nk_sum and the backward-broadcast reduction kernel.
// (nk_unary and nk_scalar_binary live in nk_ew_unary.cu; the forward kernels in nk_ew_kernels.cuh.)
//
// Compiled with -fmad=false (see nk_scalarfun.cuh).

#include "nk_ew_kernels.cuh"

using namespace nkew;

namespace {

// forward + - * / with compile-time functors, everything else through the run-time functor
template <class T, int FAMILY>
int launch_binary(nk_ctx* ctx, int op, int d, T* out, const T* a, const T* b, const EwPlan& p) {
    if (d < 0) {
        switch (op) {
            case NK_OP_ADD: return launch_ew<T, 2>(ctx, out, a, b, p, BinFix<T, NK_OP_ADD>{});
            case NK_OP_SUB: return launch_ew<T, 2>(ctx, out, a, b, p, BinFix<T, NK_OP_SUB>{});
            case NK_OP_MUL: return launch_ew<T, 2>(ctx, out, a, b, p, BinFix<T, NK_OP_MUL>{});
            case NK_OP_DIV: return launch_ew<T, 2>(ctx, out, a, b, p, BinFix<T, NK_OP_DIV>{});
            default: break;
        }
    }
    return launch_ew<T, 2>(ctx, out, a, b, p, BinF<T, FAMILY>{op, d});
}

// ---- broadcast backward: reduction over the dims where the origin is smaller -------------------------
struct RedPlan {
    int rank;
    int64_t total;                  // origin elements
    int64_t odiv[NK_MAX_RANK];      // decode of the origin's flat index
    int64_t s0[NK_MAX_RANK];        // origin strides
    int64_t p1[NK_MAX_RANK], p2[NK_MAX_RANK];  // handle/drain stride applied to the origin index
    int nred;
    int64_t rext[NK_MAX_RANK], r1[NK_MAX_RANK], r2[NK_MAX_RANK];  // reduced dims: extent, handle stride, drain stride
    int64_t b0, b1, b2;
};

// One thread per origin element; the reduction runs with the lowest reduced dim fastest, the order of
// the state machine in CPUBroadcast.java:118-150, so F32 results match the CPU bit for bit.
template <class T>
__global__ void __launch_bounds__(256) nk_broadcast_reduce_kernel(T* __restrict__ t0, const T* __restrict__ t1, const T* __restrict__ t2,
                                                                  RedPlan p, int op, int d) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
        int64_t rem = i, o0 = p.b0, o1 = p.b1, o2 = p.b2;
        for (int k = 0; k < p.rank; k++) {
            int64_t idx = rem / p.odiv[k];
            rem -= idx * p.odiv[k];
            o0 += idx * p.s0[k]; o1 += idx * p.p1[k]; o2 += idx * p.p2[k];
        }
        T value = 0;
        if (p.nred == 0) {
            value += nkf::bin<0>(op, d, t1[o1], t2[o2]);
        } else if (p.nred == 1) {
            for (int64_t r = 0; r < p.rext[0]; r++) value += nkf::bin<0>(op, d, t1[o1 + r * p.r1[0]], t2[o2 + r * p.r2[0]]);
        } else {
            int64_t q[NK_MAX_RANK];
            for (int k = 0; k < p.nred; k++) q[k] = 0;
            int64_t c1 = o1, c2 = o2;
            while (true) {
                value += nkf::bin<0>(op, d, t1[c1], t2[c2]);
                int k = 0;
                for (; k < p.nred; k++) {
                    q[k]++; c1 += p.r1[k]; c2 += p.r2[k];
                    if (q[k] < p.rext[k]) break;
                    c1 -= q[k] * p.r1[k]; c2 -= q[k] * p.r2[k]; q[k] = 0;
                }
                if (k == p.nred) break;
            }
        }
        t0[o0] = value;
    }
}

// Vectorised variant: the innermost dim is not reduced and all three tensors are unit-stride (the handle may be
// broadcast) along it, so a thread owns one 128-bit vector of origin elements and every step of its reduction
// loop is one 128-bit load per operand. The summation order per element is unchanged (lowest reduced dim
// fastest), hence still bit-identical to the CPU for + - *. OP/D are compile-time for the common operators.
template <class T, int OP, int D>
__global__ void __launch_bounds__(256) nk_broadcast_reduce_vec_kernel(T* __restrict__ t0, const T* __restrict__ t1, const T* __restrict__ t2,
                                                                      RedPlan p, int64_t total_vec, int handle_inner) {
    using V = typename Vec4<T>::type;
    constexpr int N = Vec4<T>::N;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t v = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; v < total_vec; v += stride) {
        int64_t rem = v * N, o0 = p.b0, o1 = p.b1, o2 = p.b2;
        for (int k = 0; k < p.rank; k++) {
            int64_t idx = rem / p.odiv[k];
            rem -= idx * p.odiv[k];
            o0 += idx * p.s0[k]; o1 += idx * p.p1[k]; o2 += idx * p.p2[k];
        }
        T acc[N];
#pragma unroll
        for (int k = 0; k < N; k++) acc[k] = T(0);
        int64_t q[NK_MAX_RANK];
        for (int k = 0; k < p.nred; k++) q[k] = 0;
        const int64_t n0 = p.nred > 0 ? p.rext[0] : 1, a0 = p.nred > 0 ? p.r1[0] : 0, b0 = p.nred > 0 ? p.r2[0] : 0;
        int64_t c1 = o1, c2 = o2;
        while (true) {
            // lowest reduced dim as a plain loop, 4 steps fetched ahead of the (ordered) additions
            for (int64_t r = 0; r < n0; r += 4) {
                T hv[4][N], dv[4][N];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (r + u < n0) {
                        *reinterpret_cast<V*>(dv[u]) = __ldcs(reinterpret_cast<const V*>(t2 + c2 + (r + u) * b0));
                        if (handle_inner) *reinterpret_cast<V*>(hv[u]) = __ldg(reinterpret_cast<const V*>(t1 + c1 + (r + u) * a0));
                        else { T h = t1[c1 + (r + u) * a0]; for (int k = 0; k < N; k++) hv[u][k] = h; }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    if (r + u < n0) {
#pragma unroll
                        for (int k = 0; k < N; k++) acc[k] += nkf::bin<0>(OP, D, hv[u][k], dv[u][k]);
                    }
                }
            }
            int k = 1;
            for (; k < p.nred; k++) {
                q[k]++; c1 += p.r1[k]; c2 += p.r2[k];
                if (q[k] < p.rext[k]) break;
                c1 -= q[k] * p.r1[k]; c2 -= q[k] * p.r2[k]; q[k] = 0;
            }
            if (k >= p.nred) break;
        }
        *reinterpret_cast<V*>(t0 + o0) = *reinterpret_cast<V*>(acc);
    }
}

template <class T>
bool try_reduce_vec(nk_ctx* ctx, T* t0, const T* t1, const T* t2, const RedPlan& p, int op, int d, const NkView& v0, int* status) {
    constexpr int N = Vec4<T>::N;
    const int last = p.rank - 1;
    if (p.nred < 1 || !v0.imap_row_major) return false;
    // innermost dim: kept (not reduced), unit stride in origin and drain, unit or zero stride in the handle
    if (p.s0[last] != 1 || p.p2[last] != 1 || (p.p1[last] != 1 && p.p1[last] != 0)) return false;
    if (v0.shape[last] % N) return false;
    auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    if (!al(t0 + p.b0) || !al(t1 + p.b1) || !al(t2 + p.b2)) return false;
    for (int k = 0; k < last; k++)
        if (p.s0[k] % N || p.p1[k] % N || p.p2[k] % N) return false;
    for (int k = 0; k < p.nred; k++)
        if (p.r1[k] % N || p.r2[k] % N) return false;
    const int64_t total_vec = p.total / N;
    const int hi = p.p1[last] == 1 ? 1 : 0;
    int block = 256, grid = nk_grid_for(ctx, total_vec, block, 8);
#define NK_RED(OPC, DC) nk_broadcast_reduce_vec_kernel<T, OPC, DC><<<grid, block, 0, ctx->stream>>>(t0, t1, t2, p, total_vec, hi)
    if (op == NK_OP_MUL_BOTH) NK_RED(NK_OP_MUL_BOTH, 0);
    else if (op == NK_OP_ADD) NK_RED(NK_OP_ADD, 0);
    else if (op == NK_OP_SUB && d == 0) NK_RED(NK_OP_SUB, 0);
    else if (op == NK_OP_SUB && d == 1) NK_RED(NK_OP_SUB, 1);
    else if (op == NK_OP_MUL && d == 0) NK_RED(NK_OP_MUL, 0);
    else if (op == NK_OP_MUL && d == 1) NK_RED(NK_OP_MUL, 1);
    else return false;
#undef NK_RED
    *status = nk_after_launch(ctx, "nk_broadcast_reduce_vec_kernel");
    return true;
}

// ---- fill with fun(value) ---------------------------------------------------------------------------
template <class T>
__global__ void __launch_bounds__(256) nk_fill_fun_kernel(T* __restrict__ out, EwPlan p, int fun, bool derive, T value) {
    const T v = nkf::fun(fun, derive, value);
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
        int64_t rem = i, o0 = p.b0;
        for (int k = 0; k < p.nd; k++) {
            int64_t idx = rem / p.div[k];
            rem -= idx * p.div[k];
            o0 += idx * p.s0[k];
        }
        out[o0] = v;
    }
}

// ---- sum: 128-wide tiles, recursively, in CPUSum's order ----------------------------------------------
// level 0 gathers through the view; one thread adds the 128 elements of its tile in index order.
template <class T>
__global__ void __launch_bounds__(128) nk_sum_tiles_kernel(const T* __restrict__ in, EwPlan p, bool through_view, int64_t n,
                                                           T* __restrict__ out, int64_t n_tiles) {
    __shared__ T tile[4][128 + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // each warp stages one tile at a time (coalesced), lane 0 then adds it up in order
    for (int64_t t = int64_t(blockIdx.x) * 4 + warp; t < n_tiles; t += int64_t(gridDim.x) * 4) {
        const int64_t off = t * 128;
        const int64_t lim = (off + 128 < n) ? 128 : (n - off);
        for (int k = lane; k < lim; k += 32) {
            int64_t i = off + k, src = i;
            if (through_view) {
                int64_t rem = i; src = p.b0;
                for (int j = 0; j < p.nd; j++) { int64_t idx = rem / p.div[j]; rem -= idx * p.div[j]; src += idx * p.s0[j]; }
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

}  // namespace

// ------------------------------------------------------------------------------------------------
// entry points
// ------------------------------------------------------------------------------------------------
extern "C" int nk_broadcast(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                            nk_buf* drn, const int32_t* cfg0, nk_buf* a, const int32_t* cfg1, nk_buf* b, const int32_t* cfg2,
                            int32_t d) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64)  // CPUBroadcast.java:46-56 supports exactly these two
        return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_broadcast: dtype %d not supported (F32/F64 only)", dtype);
    if (!known_op(op, false, true)) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast: unknown op %d", op);
    NkView v0, v1, v2;
    int st;
    if ((st = nk_view_parse(ctx, "nk_broadcast(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    if ((st = nk_view_parse(ctx, "nk_broadcast(src1)", a, cfg1, rank, dtype, &v1))) return st;
    if ((st = nk_view_parse(ctx, "nk_broadcast(src2)", b, cfg2, rank, dtype, &v2))) return st;
    if (d < 0) {
        bool f1[NK_MAX_RANK], f2[NK_MAX_RANK];
        for (int k = 0; k < rank; k++) {
            // CPUBroadcast.java:82-93: equal shapes -> both follow; otherwise the larger follows, the smaller stays at 0
            f1[k] = v1.shape[k] >= v2.shape[k];
            f2[k] = v2.shape[k] >= v1.shape[k];
            int64_t big = v1.shape[k] > v2.shape[k] ? v1.shape[k] : v2.shape[k];
            if (v0.shape[k] > big)
                return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast: drain dim %d = %lld exceeds both sources (%lld, %lld)", k,
                               (long long)v0.shape[k], (long long)v1.shape[k], (long long)v2.shape[k]);
        }
        EwPlan p;
        make_plan(v0, &v1, f1, &v2, f2, &p);
        if (dtype == NK_F32) return launch_binary<float, 0>(ctx, op, -1, data_of<float>(drn), data_of<float>(a), data_of<float>(b), p);
        return launch_binary<double, 0>(ctx, op, -1, data_of<double>(drn), data_of<double>(a), data_of<double>(b), p);
    }
    // d >= 0: (origin t0, handle t1, drain t2), CPUBroadcast.java:99-158
    if (d > 1) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast: derivative index %d, expected 0 or 1", d);
    RedPlan p;
    p.rank = rank;
    p.total = v0.size;
    p.nred = 0;
    p.b0 = v0.base; p.b1 = v1.base; p.b2 = v2.base;
    for (int k = 0; k < rank; k++) {
        p.odiv[k] = v0.imap[k];
        p.s0[k] = v0.estride[k];
        int64_t s0 = v0.shape[k], s1 = v1.shape[k], s2 = v2.shape[k];
        if (s0 == s1) {
            if (s2 != 1 && s2 < s0)
                return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast(d>=0): dim %d: drain extent %lld smaller than origin %lld", k, (long long)s2, (long long)s0);
            p.p1[k] = v1.estride[k];
            p.p2[k] = (s2 == 1) ? 0 : v2.estride[k];
        } else if (s0 > s1) {
            if (s2 < s0) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast(d>=0): dim %d: drain extent %lld smaller than origin %lld", k, (long long)s2, (long long)s0);
            p.p1[k] = 0;
            p.p2[k] = v2.estride[k];
        } else {  // s0 < s1: summed over the handle's extent, handle and drain advance together
            if (s0 != 1) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_broadcast(d>=0): dim %d: origin extent %lld must be 1 where the handle (%lld) is larger", k, (long long)s0, (long long)s1);
            if (s2 < s1) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_broadcast(d>=0): dim %d: drain extent %lld smaller than handle %lld", k, (long long)s2, (long long)s1);
            p.p1[k] = 0; p.p2[k] = 0;
            p.rext[p.nred] = s1; p.r1[p.nred] = v1.estride[k]; p.r2[p.nred] = v2.estride[k];
            p.nred++;
        }
    }
    {
        int vst = NK_OK;
        bool done = (dtype == NK_F32) ? try_reduce_vec<float>(ctx, data_of<float>(drn), data_of<float>(a), data_of<float>(b), p, op, d, v0, &vst)
                                      : try_reduce_vec<double>(ctx, data_of<double>(drn), data_of<double>(a), data_of<double>(b), p, op, d, v0, &vst);
        if (done) return vst;
    }
    int block = 256, grid = nk_grid_for(ctx, p.total, block, 8);
    if (dtype == NK_F32) nk_broadcast_reduce_kernel<float><<<grid, block, 0, ctx->stream>>>(data_of<float>(drn), data_of<float>(a), data_of<float>(b), p, op, d);
    else nk_broadcast_reduce_kernel<double><<<grid, block, 0, ctx->stream>>>(data_of<double>(drn), data_of<double>(a), data_of<double>(b), p, op, d);
    return nk_after_launch(ctx, "nk_broadcast_reduce_kernel");
}

extern "C" int nk_binary(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                         nk_buf* drn, const int32_t* cfg0, nk_buf* a, const int32_t* cfg1, nk_buf* b, const int32_t* cfg2,
                         int32_t d) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_binary: dtype %d not supported (F32/F64 only)", dtype);
    if (!known_op(op, false, false)) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_binary: unknown op %d", op);
    NkView v0, v1, v2;
    int st;
    if ((st = nk_view_parse(ctx, "nk_binary(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    if ((st = nk_view_parse(ctx, "nk_binary(src1)", a, cfg1, rank, dtype, &v1))) return st;
    if ((st = nk_view_parse(ctx, "nk_binary(src2)", b, cfg2, rank, dtype, &v2))) return st;
    for (int k = 0; k < rank; k++)
        if (v0.shape[k] != v1.shape[k] || v0.shape[k] != v2.shape[k])
            return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_binary: shapes differ at dim %d (%lld, %lld, %lld)", k,
                           (long long)v0.shape[k], (long long)v1.shape[k], (long long)v2.shape[k]);
    EwPlan p;
    make_plan(v0, &v1, nullptr, &v2, nullptr, &p);
    int dd = d < 0 ? -1 : d;
    if (dtype == NK_F32) return launch_binary<float, 1>(ctx, op, dd, data_of<float>(drn), data_of<float>(a), data_of<float>(b), p);
    return launch_binary<double, 1>(ctx, op, dd, data_of<double>(drn), data_of<double>(a), data_of<double>(b), p);
}

extern "C" int nk_fill_fun(nk_ctx* ctx, int32_t fun, int32_t dtype, int32_t rank, nk_buf* drn, const int32_t* cfg0,
                           double value, int32_t d) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fill_fun: dtype %d not supported (F32/F64 only)", dtype);
    if (fun < 0 || fun >= NK_FUN_COUNT) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fill_fun: unknown function id %d", fun);
    NkView v0;
    int st;
    if ((st = nk_view_parse(ctx, "nk_fill_fun(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    EwPlan p;
    make_plan(v0, nullptr, nullptr, nullptr, nullptr, &p);
    int block = 256, grid = nk_grid_for(ctx, p.total, block, 8);
    if (dtype == NK_F32) nk_fill_fun_kernel<float><<<grid, block, 0, ctx->stream>>>(data_of<float>(drn), p, fun, d >= 0, float(value));
    else nk_fill_fun_kernel<double><<<grid, block, 0, ctx->stream>>>(data_of<double>(drn), p, fun, d >= 0, value);
    return nk_after_launch(ctx, "nk_fill_fun_kernel");
}

template <class T>
static int sum_impl(nk_ctx* ctx, const T* in, const EwPlan& p, int64_t n, T* out_elem) {
    // level sizes: n -> ceil(n/128) -> ... -> 1 ; ping-pong inside the ctx scratch block
    int64_t n1 = (n + 127) / 128;
    int64_t n2 = (n1 + 127) / 128;
    void* scratch = nullptr;
    int st = nk_scratch(ctx, size_t(n1 + n2 + 2) * sizeof(T), &scratch);
    if (st) return st;
    T* bufA = reinterpret_cast<T*>(scratch);
    T* bufB = bufA + n1 + 1;
    const T* src = in;
    int64_t cur = n;
    bool through_view = true;
    T* dst = bufA;
    if (cur == 1) {
        // CPUSum returns the input itself for a single element
        nk_sum_tiles_kernel<T><<<1, 128, 0, ctx->stream>>>(src, p, true, 1, out_elem, 1);
        return nk_after_launch(ctx, "nk_sum_tiles_kernel");
    }
    while (true) {
        int64_t tiles = (cur + 127) / 128;
        T* target = (tiles == 1) ? out_elem : dst;
        int64_t want = (tiles + 3) / 4;
        int64_t cap = int64_t(ctx->prop.multiProcessorCount) * 16;
        int grid = int(want < cap ? want : cap);
        nk_sum_tiles_kernel<T><<<grid, 128, 0, ctx->stream>>>(src, p, through_view, cur, target, tiles);
        st = nk_after_launch(ctx, "nk_sum_tiles_kernel");
        if (st) return st;
        if (tiles == 1) break;
        src = target;
        through_view = false;
        cur = tiles;
        dst = (dst == bufA) ? bufB : bufA;
    }
    return NK_OK;
}

extern "C" int nk_sum(nk_ctx* ctx, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out, int64_t out_index) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_sum: dtype %d not supported (F32/F64 only)", dtype);
    NkView v;
    int st;
    if ((st = nk_view_parse(ctx, "nk_sum(src)", src, cfg, rank, dtype, &v))) return st;
    if (out == nullptr || out->magic != 0x4e4b4246 || out->dtype != dtype) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_sum: invalid output buffer");
    if (out->device != ctx->device)
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_sum: output buffer lives on device %d, context on device %d", out->device, ctx->device);
    if (out_index < 0 || out_index >= out->n_elems) return nk_fail(ctx, NK_ERR_BOUNDS, "nk_sum: output index %lld outside the buffer", (long long)out_index);
    EwPlan p;
    make_plan(v, nullptr, nullptr, nullptr, nullptr, &p);
    if (dtype == NK_F32) return sum_impl<float>(ctx, data_of<float>(src), p, v.size, data_of<float>(out) + out_index);
    return sum_impl<double>(ctx, data_of<double>(src), p, v.size, data_of<double>(out) + out_index);
}
