// Broadcast / elementwise / scalar / fill / sum kernels.
//
// All of these are HBM-bound streaming kernels: one pass, every input element read once and every
// output element written once. The host turns the three NDConfiguration views into one iteration plan
// (per-dimension divisor + one element stride per tensor, broadcast dims get stride 0, adjacent dims
// are merged when all tensors allow it), passed by value in the kernel parameters, so the kernels do
// no index-map loads from memory (the reference's OpenCL templates copy 5*rank ints per tensor into
// private memory and recompute a full strided index per access, kernels/utility.cl:15-70).
//
// Compiled with -fmad=false (see nk_scalarfun.cuh).

#include "nk_internal.h"
#include "nk_scalarfun.cuh"

namespace {

struct EwPlan {
    int nd;                       // dims after merging (>= 1)
    int64_t total;                // number of drain elements
    int64_t div[NK_MAX_RANK];     // idx_k = i / div[k]; i %= div[k]
    int64_t ext[NK_MAX_RANK];     // extent of dim k (row-major plans only)
    int64_t s0[NK_MAX_RANK], s1[NK_MAX_RANK], s2[NK_MAX_RANK];
    int64_t b0, b1, b2;
    bool row_major;               // div[] are the row-major divisors of ext[]
};

// Builds the iteration plan over the drain's index space. sel1/sel2 give, per original dim, whether the
// source follows the drain index (true) or stays at 0 (false: a broadcast dim).
void make_plan(const NkView& v0, const NkView* v1, const bool* follow1, const NkView* v2, const bool* follow2, EwPlan* p) {
    int rank = v0.rank;
    p->total = v0.size;
    p->b0 = v0.base;
    p->b1 = v1 ? v1->base : 0;
    p->b2 = v2 ? v2->base : 0;
    int64_t e[NK_MAX_RANK], a0[NK_MAX_RANK], a1[NK_MAX_RANK], a2[NK_MAX_RANK];
    for (int k = 0; k < rank; k++) {
        e[k] = v0.shape[k];
        a0[k] = v0.estride[k];
        a1[k] = (v1 && (!follow1 || follow1[k])) ? v1->estride[k] : 0;
        a2[k] = (v2 && (!follow2 || follow2[k])) ? v2->estride[k] : 0;
    }
    if (!v0.imap_row_major) {
        // Decode with the drain's own indicesMap, exactly as NDConfiguration.indicesOfIndex does.
        p->nd = rank;
        p->row_major = false;
        for (int k = 0; k < rank; k++) {
            p->div[k] = v0.imap[k]; p->ext[k] = e[k];
            p->s0[k] = a0[k]; p->s1[k] = a1[k]; p->s2[k] = a2[k];
        }
        return;
    }
    // drop size-1 dims, merge neighbours (outer k with inner k+1) when every tensor is linear across them
    int nd = 0;
    for (int k = 0; k < rank; k++) {
        if (e[k] == 1) continue;
        if (nd > 0 && p->s0[nd - 1] == e[k] * a0[k] && p->s1[nd - 1] == e[k] * a1[k] && p->s2[nd - 1] == e[k] * a2[k]) {
            p->ext[nd - 1] *= e[k];
            p->s0[nd - 1] = a0[k]; p->s1[nd - 1] = a1[k]; p->s2[nd - 1] = a2[k];
        } else {
            p->ext[nd] = e[k];
            p->s0[nd] = a0[k]; p->s1[nd] = a1[k]; p->s2[nd] = a2[k];
            nd++;
        }
    }
    if (nd == 0) { p->ext[0] = 1; p->s0[0] = p->s1[0] = p->s2[0] = 0; nd = 1; }
    p->nd = nd;
    p->row_major = true;
    int64_t d = 1;
    for (int k = nd - 1; k >= 0; k--) { p->div[k] = d; d *= p->ext[k]; }
}

// ---- functors -------------------------------------------------------------------------------------
template <class T> struct UnaryF {
    int f; bool derive;
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::fun(f, derive, a); }
};
template <class T, int FAMILY> struct BinF {
    int op, d;
    __device__ __forceinline__ T operator()(T a, T b) const { return nkf::bin<FAMILY>(op, d, a, b); }
};
template <class T> struct ScalarF {
    int op, d; T value;
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::bin<2>(op, d, a, value); }
};

template <class T> struct Vec4 { using type = float4; static constexpr int N = 4; };
template <> struct Vec4<double> { using type = double2; static constexpr int N = 2; };

// ---- kernel 1: fully contiguous, 128-bit accesses ---------------------------------------------------
// All tensors are linear with element stride 1 (sources may have stride 0 = a broadcast scalar).
template <class T, int NIN, class F>
__global__ void __launch_bounds__(256) nk_ew_linear_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                           int64_t n, int sa, int sb, F f) {
    using V = typename Vec4<T>::type;
    constexpr int N = Vec4<T>::N;
    const int64_t nvec = n / N;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    for (int64_t i = tid; i < nvec; i += stride) {
        T av[N], bv[N], ov[N];
        if (sa) *reinterpret_cast<V*>(av) = __ldcs(reinterpret_cast<const V*>(a) + i);
        else { T s = a[0]; for (int k = 0; k < N; k++) av[k] = s; }
        if (NIN == 2) {
            if (sb) *reinterpret_cast<V*>(bv) = __ldcs(reinterpret_cast<const V*>(b) + i);
            else { T s = b[0]; for (int k = 0; k < N; k++) bv[k] = s; }
        }
#pragma unroll
        for (int k = 0; k < N; k++) ov[k] = f(av[k], NIN == 2 ? bv[k] : T(0));
        __stcs(reinterpret_cast<V*>(out) + i, *reinterpret_cast<V*>(ov));
    }
    for (int64_t i = nvec * N + tid; i < n; i += stride)
        out[i] = f(a[sa ? i : 0], NIN == 2 ? b[sb ? i : 0] : T(0));
}

// ---- kernel 2: rows ---------------------------------------------------------------------------------
// The innermost merged dim is long and every tensor has stride 1 or 0 along it. A CTA walks rows
// (all outer dims, decoded once per row) and streams the row with 128-bit accesses when VEC.
template <class T, int NIN, class F, bool VEC>
__global__ void __launch_bounds__(256) nk_ew_rows_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                         EwPlan p, int64_t rows, int64_t inner, F f) {
    using V = typename Vec4<T>::type;
    constexpr int N = Vec4<T>::N;
    const int last = p.nd - 1;
    const int sa = int(p.s1[last]), sb = int(p.s2[last]);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int64_t rem = r, o0 = p.b0, o1 = p.b1, o2 = p.b2;
        for (int k = 0; k < last; k++) {
            int64_t dk = p.div[k] / inner;  // divisor in units of rows
            int64_t idx = rem / dk;
            rem -= idx * dk;
            o0 += idx * p.s0[k]; o1 += idx * p.s1[k]; o2 += idx * p.s2[k];
        }
        T* orow = out + o0;
        const T* arow = a + o1;
        const T* brow = (NIN == 2) ? b + o2 : nullptr;
        if (VEC) {
            const int64_t nvec = inner / N;
            for (int64_t i = threadIdx.x; i < nvec; i += blockDim.x) {
                T av[N], bv[N], ov[N];
                if (sa) *reinterpret_cast<V*>(av) = __ldg(reinterpret_cast<const V*>(arow) + i);
                else { T s = arow[0]; for (int k = 0; k < N; k++) av[k] = s; }
                if (NIN == 2) {
                    if (sb) *reinterpret_cast<V*>(bv) = __ldg(reinterpret_cast<const V*>(brow) + i);
                    else { T s = brow[0]; for (int k = 0; k < N; k++) bv[k] = s; }
                }
#pragma unroll
                for (int k = 0; k < N; k++) ov[k] = f(av[k], NIN == 2 ? bv[k] : T(0));
                __stcs(reinterpret_cast<V*>(orow) + i, *reinterpret_cast<V*>(ov));
            }
        } else {
            for (int64_t i = threadIdx.x; i < inner; i += blockDim.x)
                orow[i] = f(arow[sa ? i : 0], NIN == 2 ? brow[sb ? i : 0] : T(0));
        }
    }
}

// ---- kernel 3: flat, any view -----------------------------------------------------------------------
template <class T, int NIN, class F>
__global__ void __launch_bounds__(256) nk_ew_flat_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                         EwPlan p, F f) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < p.total; i += stride) {
        int64_t rem = i, o0 = p.b0, o1 = p.b1, o2 = p.b2;
        for (int k = 0; k < p.nd; k++) {
            int64_t idx = rem / p.div[k];
            rem -= idx * p.div[k];
            o0 += idx * p.s0[k]; o1 += idx * p.s1[k]; o2 += idx * p.s2[k];
        }
        out[o0] = f(a[o1], NIN == 2 ? b[o2] : T(0));
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <class T, int NIN, class F>
int launch_ew(nk_ctx* ctx, T* out, const T* a, const T* b, const EwPlan& p, F f) {
    constexpr int N = Vec4<T>::N;
    const int block = 256;
    const int last = p.nd - 1;
    const bool inner_ok = p.row_major && p.s0[last] == 1 && (p.s1[last] == 1 || p.s1[last] == 0) &&
                          (NIN == 1 || p.s2[last] == 1 || p.s2[last] == 0);
    if (inner_ok && p.nd == 1) {
        T* o = out + p.b0;
        const T* pa = a + p.b1;
        const T* pb = NIN == 2 ? b + p.b2 : nullptr;
        // 128-bit path needs all streamed pointers 16-byte aligned
        bool al = aligned16(o) && (p.s1[0] == 0 || aligned16(pa)) && (NIN == 1 || p.s2[0] == 0 || aligned16(pb));
        if (al) {
            int grid = nk_grid_for(ctx, (p.total + N - 1) / N, block, 16);
            nk_ew_linear_kernel<T, NIN, F><<<grid, block, 0, ctx->stream>>>(o, pa, pb, p.total, int(p.s1[0]), int(p.s2[0]), f);
            return nk_after_launch(ctx, "nk_ew_linear_kernel");
        }
    }
    if (inner_ok && p.nd > 1 && p.ext[last] >= 128) {
        const int64_t inner = p.ext[last];
        const int64_t rows = p.total / inner;
        bool vec = (inner % N == 0) && aligned16(out + p.b0) && aligned16(a + p.b1) && (NIN == 1 || aligned16(b + p.b2));
        for (int k = 0; k < last && vec; k++)
            vec = (p.s0[k] % N == 0) && (p.s1[k] % N == 0) && (NIN == 1 || p.s2[k] % N == 0);
        int64_t cap = int64_t(ctx->prop.multiProcessorCount) * 16;
        int grid = int(rows < cap ? rows : cap);
        if (vec) nk_ew_rows_kernel<T, NIN, F, true><<<grid, block, 0, ctx->stream>>>(out, a, b, p, rows, inner, f);
        else nk_ew_rows_kernel<T, NIN, F, false><<<grid, block, 0, ctx->stream>>>(out, a, b, p, rows, inner, f);
        return nk_after_launch(ctx, "nk_ew_rows_kernel");
    }
    int grid = nk_grid_for(ctx, p.total, block, 16);
    nk_ew_flat_kernel<T, NIN, F><<<grid, block, 0, ctx->stream>>>(out, a, b, p, f);
    return nk_after_launch(ctx, "nk_ew_flat_kernel");
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

template <class T> T* data_of(nk_buf* b) { return reinterpret_cast<T*>(b->ptr); }

bool known_op(int op, bool allow_idy, bool allow_both) {
    if (op >= NK_OP_ADD && op <= NK_OP_POW) return true;
    if (op == NK_OP_IDY) return allow_idy;
    if (op == NK_OP_MUL_BOTH) return allow_both;
    return false;
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
        if (dtype == NK_F32) return launch_ew<float, 2>(ctx, data_of<float>(drn), data_of<float>(a), data_of<float>(b), p, BinF<float, 0>{op, -1});
        return launch_ew<double, 2>(ctx, data_of<double>(drn), data_of<double>(a), data_of<double>(b), p, BinF<double, 0>{op, -1});
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
    if (dtype == NK_F32) return launch_ew<float, 2>(ctx, data_of<float>(drn), data_of<float>(a), data_of<float>(b), p, BinF<float, 1>{op, dd});
    return launch_ew<double, 2>(ctx, data_of<double>(drn), data_of<double>(a), data_of<double>(b), p, BinF<double, 1>{op, dd});
}

extern "C" int nk_unary(nk_ctx* ctx, int32_t fun, int32_t dtype, int32_t rank,
                        nk_buf* drn, const int32_t* cfg0, nk_buf* src, const int32_t* cfg1, int32_t d) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_unary: dtype %d not supported (F32/F64 only)", dtype);
    if (fun < 0 || fun >= NK_FUN_COUNT) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_unary: unknown function id %d", fun);
    NkView v0, v1;
    int st;
    if ((st = nk_view_parse(ctx, "nk_unary(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    if ((st = nk_view_parse(ctx, "nk_unary(src)", src, cfg1, rank, dtype, &v1))) return st;
    for (int k = 0; k < rank; k++)
        if (v0.shape[k] != v1.shape[k])
            return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_unary: shapes differ at dim %d (%lld vs %lld)", k, (long long)v0.shape[k], (long long)v1.shape[k]);
    EwPlan p;
    make_plan(v0, &v1, nullptr, nullptr, nullptr, &p);
    if (dtype == NK_F32) return launch_ew<float, 1>(ctx, data_of<float>(drn), data_of<float>(src), (const float*)nullptr, p, UnaryF<float>{fun, d >= 0});
    return launch_ew<double, 1>(ctx, data_of<double>(drn), data_of<double>(src), (const double*)nullptr, p, UnaryF<double>{fun, d >= 0});
}

extern "C" int nk_scalar_binary(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                                nk_buf* drn, const int32_t* cfg0, nk_buf* src, const int32_t* cfg1, double value, int32_t d) {
    NK_CHECK_CTX(ctx);
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_scalar_binary: dtype %d not supported (F32/F64 only)", dtype);
    if (!known_op(op, true, false)) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_scalar_binary: unknown op %d", op);
    NkView v0, v1;
    int st;
    if ((st = nk_view_parse(ctx, "nk_scalar_binary(drain)", drn, cfg0, rank, dtype, &v0))) return st;
    if ((st = nk_view_parse(ctx, "nk_scalar_binary(src)", src, cfg1, rank, dtype, &v1))) return st;
    for (int k = 0; k < rank; k++)
        if (v0.shape[k] != v1.shape[k])
            return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_scalar_binary: shapes differ at dim %d (%lld vs %lld)", k, (long long)v0.shape[k], (long long)v1.shape[k]);
    EwPlan p;
    make_plan(v0, &v1, nullptr, nullptr, nullptr, &p);
    int dd = d < 0 ? -1 : d;
    if (dtype == NK_F32) return launch_ew<float, 1>(ctx, data_of<float>(drn), data_of<float>(src), (const float*)nullptr, p, ScalarF<float>{op, dd, float(value)});
    return launch_ew<double, 1>(ctx, data_of<double>(drn), data_of<double>(src), (const double*)nullptr, p, ScalarF<double>{op, dd, value});
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
    if (out_index < 0 || out_index >= out->n_elems) return nk_fail(ctx, NK_ERR_BOUNDS, "nk_sum: output index %lld outside the buffer", (long long)out_index);
    EwPlan p;
    make_plan(v, nullptr, nullptr, nullptr, nullptr, &p);
    if (dtype == NK_F32) return sum_impl<float>(ctx, data_of<float>(src), p, v.size, data_of<float>(out) + out_index);
    return sum_impl<double>(ctx, data_of<double>(src), p, v.size, data_of<double>(out) + out_index);
}
