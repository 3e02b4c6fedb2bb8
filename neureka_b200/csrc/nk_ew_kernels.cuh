// Forward kernels of the broadcast / elementwise / scalar family and the plan they consume.
//
// All of these are HBM-bound streaming kernels: one pass, every input element read once and every output
// element written once. The host turns the NDConfiguration views of a call into one iteration plan
// (per-dimension divisor + one element stride per tensor, broadcast dims get stride 0, adjacent dims are
// merged when all tensors allow it), passed by value in the kernel parameters, so the kernels do no index-map
// loads from memory (the reference's OpenCL templates copy 5*rank ints per tensor into private memory and
// recompute a full strided index per access, kernels/utility.cl:15-70).
//
// The scalar operation is a functor. Hot operations (+ - * / forward, the common activations) are
// compile-time functors, so the per-element work is the operation's own instructions; everything else goes
// through run-time functors that switch on the operation id (uniform branch).
//
// Translation units including this header are compiled with -fmad=false (see nk_scalarfun.cuh).
#pragma once
#include "nk_internal.h"
#include "nk_scalarfun.cuh"

namespace nkew {

struct EwPlan {
    int nd;                       // dims after merging (>= 1)
    int64_t total;                // number of drain elements
    int64_t div[NK_MAX_RANK];     // idx_k = i / div[k]; i %= div[k]
    int64_t ext[NK_MAX_RANK];     // extent of dim k (row-major plans only)
    int64_t s0[NK_MAX_RANK], s1[NK_MAX_RANK], s2[NK_MAX_RANK];
    int64_t b0, b1, b2;
    bool row_major;               // div[] are the row-major divisors of ext[]
};

// Builds the iteration plan over the drain's index space. follow1/follow2 give, per original dim, whether
// the source follows the drain index (true) or stays at 0 (false: a broadcast dim); null = follows everywhere.
inline void make_plan(const NkView& v0, const NkView* v1, const bool* follow1, const NkView* v2, const bool* follow2, EwPlan* p) {
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
template <class T> struct UnaryF {            // run-time function id
    int f; bool derive;
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::fun(f, derive, a); }
};
template <class T, int FUN, bool DERIVE> struct UnaryFix {   // compile-time function id: the switch folds away
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::fun(FUN, DERIVE, a); }
};
template <class T, int FAMILY> struct BinF {  // run-time operator id
    int op, d;
    __device__ __forceinline__ T operator()(T a, T b) const { return nkf::bin<FAMILY>(op, d, a, b); }
};
template <class T, int OP> struct BinFix {    // forward + - * / (identical in the Broadcast and BiElementwise families)
    __device__ __forceinline__ T operator()(T a, T b) const { return nkf::bin<1>(OP, -1, a, b); }
};
template <class T> struct ScalarF {
    int op, d; T value;
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::bin<2>(op, d, a, value); }
};
template <class T, int OP> struct ScalarFix {
    T value;
    __device__ __forceinline__ T operator()(T a, T) const { return nkf::bin<2>(OP, -1, a, value); }
};

// Functors whose function has a straight-line form for all but a few inputs: the kernels evaluate fast() for every element
// of a vector first and repair the rare ones afterwards (see tanh32_fast in nk_scalarfun.cuh for why).
template <class F> struct TwoPhase { static constexpr bool value = false; };
template <int FUN, bool DERIVE> struct TwoPhase<UnaryFix<float, FUN, DERIVE>> {
    // tanh (and its derivative): fast form + literal repair; sig, silu, gelu forward: straight-line already, they only want
    // the kernel loop that keeps the next loads in flight under their arithmetic
    static constexpr bool value = FUN == NK_FUN_TANH || (!DERIVE && (FUN == NK_FUN_SIG || FUN == NK_FUN_SILU || FUN == NK_FUN_GELU));
    static __device__ __forceinline__ float fast(float a) {
        if (FUN != NK_FUN_TANH) return nkf::fun(FUN, DERIVE, a);
        const float t = nkf::tanh32_fast(a);
        if (!DERIVE) return t;
        const double td = double(t);
        return float(1 - td * td);
    }
    static __device__ __forceinline__ bool rare(float a) { return FUN == NK_FUN_TANH && nkf::tanh32_rare(a); }
};
// out[k] = f(a[k], b[k]) for the N elements of one vector
template <class T, int N, int NIN, class F>
__device__ __forceinline__ void apply_vec(const F& f, const T* a, const T* b, T* o) {
    if constexpr (TwoPhase<F>::value) {
        bool any = false;
#pragma unroll
        for (int k = 0; k < N; k++) { o[k] = TwoPhase<F>::fast(a[k]); any = any || TwoPhase<F>::rare(a[k]); }
        if (any) {
#pragma unroll
            for (int k = 0; k < N; k++)
                if (TwoPhase<F>::rare(a[k])) o[k] = f(a[k], T(0));
        }
    } else {
#pragma unroll
        for (int k = 0; k < N; k++) o[k] = f(a[k], NIN == 2 ? b[k] : T(0));
    }
}

template <class T> struct Vec4 { using type = float4; static constexpr int N = 4; };
template <> struct Vec4<double> { using type = double2; static constexpr int N = 2; };

// ---- kernel 1: fully contiguous, 128-bit accesses ---------------------------------------------------
// All tensors are linear with element stride 1 (sources may have stride 0 = a broadcast scalar). Two vectors
// per thread and trip: both loads are issued before the first store.
template <class T, int NIN, class F>
__global__ void __launch_bounds__(256) nk_ew_linear_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                           int64_t n, int sa, int sb, F f) {
    using V = typename Vec4<T>::type;
    constexpr int N = Vec4<T>::N;
    const int64_t nvec = n / N;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    const int64_t tid = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
    T sa0 = sa ? T(0) : a[0], sb0 = (NIN == 2 && !sb) ? b[0] : T(0);
    if constexpr (TwoPhase<F>::value && NIN == 1) {
        // Arithmetic-heavy function (hundreds of instructions per vector): the next trip's vectors are requested before this
        // trip's arithmetic starts, so their latency passes under it (without this the kernel waited on its loads: ncu,
        // long_scoreboard 3.7 per issued instruction, FP64 pipe 61 % busy).
        if (sa) {
            V cur[2], nxt[2];
            int64_t i = tid;
            if (i < nvec) cur[0] = __ldcs(reinterpret_cast<const V*>(a) + i);
            if (i + stride < nvec) cur[1] = __ldcs(reinterpret_cast<const V*>(a) + i + stride);
            for (; i < nvec; i += 2 * stride) {
                const int64_t j = i + stride, ni = i + 2 * stride, nj = ni + stride;
                if (ni < nvec) nxt[0] = __ldcs(reinterpret_cast<const V*>(a) + ni);
                if (nj < nvec) nxt[1] = __ldcs(reinterpret_cast<const V*>(a) + nj);
                T ov[N];
                apply_vec<T, N, NIN>(f, reinterpret_cast<const T*>(&cur[0]), static_cast<const T*>(nullptr), ov);
                __stcs(reinterpret_cast<V*>(out) + i, *reinterpret_cast<V*>(ov));
                if (j < nvec) {
                    apply_vec<T, N, NIN>(f, reinterpret_cast<const T*>(&cur[1]), static_cast<const T*>(nullptr), ov);
                    __stcs(reinterpret_cast<V*>(out) + j, *reinterpret_cast<V*>(ov));
                }
                cur[0] = nxt[0]; cur[1] = nxt[1];
            }
            for (int64_t t = nvec * N + tid; t < n; t += stride) out[t] = f(a[t], T(0));
            return;
        }
    }
    for (int64_t i = tid; i < nvec; i += 2 * stride) {
        const int64_t j = i + stride;
        const bool two = j < nvec;
        T av[2][N], bv[2][N], ov[N];
        if (sa) {
            *reinterpret_cast<V*>(av[0]) = __ldcs(reinterpret_cast<const V*>(a) + i);
            if (two) *reinterpret_cast<V*>(av[1]) = __ldcs(reinterpret_cast<const V*>(a) + j);
        } else {
            for (int k = 0; k < N; k++) av[0][k] = av[1][k] = sa0;
        }
        if (NIN == 2) {
            if (sb) {
                *reinterpret_cast<V*>(bv[0]) = __ldcs(reinterpret_cast<const V*>(b) + i);
                if (two) *reinterpret_cast<V*>(bv[1]) = __ldcs(reinterpret_cast<const V*>(b) + j);
            } else {
                for (int k = 0; k < N; k++) bv[0][k] = bv[1][k] = sb0;
            }
        }
        apply_vec<T, N, NIN>(f, av[0], bv[0], ov);
        __stcs(reinterpret_cast<V*>(out) + i, *reinterpret_cast<V*>(ov));
        if (two) {
            apply_vec<T, N, NIN>(f, av[1], bv[1], ov);
            __stcs(reinterpret_cast<V*>(out) + j, *reinterpret_cast<V*>(ov));
        }
    }
    for (int64_t i = nvec * N + tid; i < n; i += stride)
        out[i] = f(a[sa ? i : 0], NIN == 2 ? b[sb ? i : 0] : T(0));
}

// ---- kernel 2: rows ---------------------------------------------------------------------------------
// The innermost merged dim is long and every tensor has stride 1 or 0 along it (the typical broadcast: the
// outer dims differ per operand, the inner one is shared). Rows are dealt to CTAs in contiguous blocks; a
// CTA decodes its first row with divisions once and then walks row by row with an odometer over the (one or
// two) outer dims -- adds and compares only. Within a row the threads stream 128-bit vectors; RPT rows are
// in flight per thread before the first store.
struct RowWalk {
    unsigned ext[2];               // extents of the outer dims (ext[1] is the faster one; unused entries = 1)
    unsigned long long rows;       // total rows
    unsigned long long rows_per_cta;
    unsigned vpr;                  // 128-bit vectors per row
};

template <class T, int NIN, class F, int N_OUTER>
__global__ void __launch_bounds__(256) nk_ew_rows_kernel(T* __restrict__ out, const T* __restrict__ a, const T* __restrict__ b,
                                                         EwPlan p, RowWalk rw, F f) {
    using V = typename Vec4<T>::type;
    constexpr int N = Vec4<T>::N;
    constexpr int RPT = 4;   // rows per trip (independent loads in flight per thread)
    const int last = p.nd - 1;   // == N_OUTER
    const bool sa = p.s1[last] != 0, sb = NIN == 2 && p.s2[last] != 0;
    // threads: tx walks the vectors of a row, ty selects the row inside a trip
    const unsigned TX = rw.vpr >= 256 ? 256u : (rw.vpr > 128 ? 256u : (rw.vpr > 64 ? 128u : (rw.vpr > 32 ? 64u : 32u)));
    const unsigned TY = 256u / TX;
    const unsigned tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const unsigned long long r_begin = (unsigned long long)blockIdx.x * rw.rows_per_cta;
    unsigned long long r_end = r_begin + rw.rows_per_cta;
    if (r_end > rw.rows) r_end = rw.rows;
    if (r_begin >= r_end) return;
    // decode the first row of this thread
    unsigned long long r = r_begin + ty;
    unsigned i0, i1;
    if (N_OUTER == 2) { i0 = unsigned(r / rw.ext[1]); i1 = unsigned(r - (unsigned long long)i0 * rw.ext[1]); }
    else { i0 = unsigned(r); i1 = 0; }
    int64_t o0 = p.b0 + int64_t(i0) * p.s0[0], o1 = p.b1 + int64_t(i0) * p.s1[0], o2 = p.b2 + int64_t(i0) * p.s2[0];
    if (N_OUTER == 2) { o0 += int64_t(i1) * p.s0[1]; o1 += int64_t(i1) * p.s1[1]; o2 += int64_t(i1) * p.s2[1]; }
    // per-row step of TY rows, and the wrap of the fast outer dim
    const int64_t st0 = int64_t(TY) * p.s0[N_OUTER - 1], st1 = int64_t(TY) * p.s1[N_OUTER - 1], st2 = int64_t(TY) * p.s2[N_OUTER - 1];
    const int64_t w0 = N_OUTER == 2 ? p.s0[0] - int64_t(rw.ext[1]) * p.s0[1] : 0;
    const int64_t w1 = N_OUTER == 2 ? p.s1[0] - int64_t(rw.ext[1]) * p.s1[1] : 0;
    const int64_t w2 = N_OUTER == 2 ? p.s2[0] - int64_t(rw.ext[1]) * p.s2[1] : 0;
    while (r < r_end) {
        int64_t q0[RPT], q1[RPT], q2[RPT];
        bool ok[RPT];
#pragma unroll
        for (int u = 0; u < RPT; u++) {
            ok[u] = r < r_end;
            q0[u] = o0; q1[u] = o1; q2[u] = o2;
            r += TY;
            o0 += st0; o1 += st1; o2 += st2;
            if (N_OUTER == 2) {
                i1 += TY;
                while (i1 >= rw.ext[1]) { i1 -= rw.ext[1]; o0 += w0; o1 += w1; o2 += w2; }   // TY <= 8 < any merged extent
            }
        }
        for (unsigned c = tx; c < rw.vpr; c += TX) {
            T av[RPT][N], bv[RPT][N];
#pragma unroll
            for (int u = 0; u < RPT; u++) {
                if (!ok[u]) continue;
                if (sa) *reinterpret_cast<V*>(av[u]) = __ldg(reinterpret_cast<const V*>(a + q1[u]) + c);
                else { T s = a[q1[u]]; for (int k = 0; k < N; k++) av[u][k] = s; }
                if (NIN == 2) {
                    if (sb) *reinterpret_cast<V*>(bv[u]) = __ldg(reinterpret_cast<const V*>(b + q2[u]) + c);
                    else { T s = b[q2[u]]; for (int k = 0; k < N; k++) bv[u][k] = s; }
                }
            }
#pragma unroll
            for (int u = 0; u < RPT; u++) {
                if (!ok[u]) continue;
                T ov[N];
                apply_vec<T, N, NIN>(f, av[u], bv[u], ov);
                __stcs(reinterpret_cast<V*>(out + q0[u]) + c, *reinterpret_cast<V*>(ov));
            }
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

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <class T, int NIN, class F>
int launch_ew(nk_ctx* ctx, T* out, const T* a, const T* b, const EwPlan& p_in, F f) {
    constexpr int N = Vec4<T>::N;
    const int block = 256;
    EwPlan p = p_in;
    // Few, very long rows (e.g. [n, m*k] + [1, m*k]) would leave most of the machine idle if a CTA had to take
    // whole rows: cut the inner dim into S segments, which become a second outer dim of all three tensors.
    if (p.row_major && p.nd == 2 && p.s0[1] == 1 && (p.s1[1] == 1 || p.s1[1] == 0) && (NIN == 1 || p.s2[1] == 1 || p.s2[1] == 0)) {
        const int64_t want_rows = int64_t(ctx->prop.multiProcessorCount) * 32 * 4;
        int64_t S = 1;
        while (p.ext[0] * S < want_rows && p.ext[1] / (S * 2) >= 1024 && p.ext[1] % (S * 2 * N) == 0) S *= 2;
        if (S > 1) {
            const int64_t seg = p.ext[1] / S;
            p.nd = 3;
            p.ext[2] = seg; p.s0[2] = p.s0[1]; p.s1[2] = p.s1[1]; p.s2[2] = p.s2[1];
            p.ext[1] = S; p.s0[1] = seg * p.s0[2]; p.s1[1] = seg * p.s1[2]; p.s2[1] = seg * p.s2[2];
            p.div[2] = 1; p.div[1] = seg; p.div[0] = seg * S;
        }
    }
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
            int grid = nk_grid_for(ctx, (p.total + 2 * N - 1) / (2 * N), block, 8);
            nk_ew_linear_kernel<T, NIN, F><<<grid, block, 0, ctx->stream>>>(o, pa, pb, p.total, int(p.s1[0]), int(p.s2[0]), f);
            return nk_after_launch(ctx, "nk_ew_linear_kernel");
        }
    }
    if (inner_ok && (p.nd == 2 || p.nd == 3) && p.ext[last] >= 64 && p.ext[last] % N == 0 && p.ext[last] / N < (int64_t(1) << 31)) {
        const int64_t inner = p.ext[last];
        const int64_t rows = p.total / inner;
        bool vec = aligned16(out + p.b0) && aligned16(a + p.b1) && (NIN == 1 || aligned16(b + p.b2));
        for (int k = 0; k < last && vec; k++)
            vec = (p.s0[k] % N == 0) && (p.s1[k] % N == 0) && (NIN == 1 || p.s2[k] % N == 0) && p.ext[k] < (int64_t(1) << 31);
        if (vec && (p.nd == 2 || p.ext[1] >= 8)) {
            RowWalk rw;
            rw.ext[0] = unsigned(p.ext[0]);
            rw.ext[1] = p.nd == 3 ? unsigned(p.ext[1]) : 1u;
            rw.rows = (unsigned long long)rows;
            rw.vpr = unsigned(inner / N);
            // enough CTAs to fill the machine several times over, each with a contiguous block of rows
            const int64_t want = int64_t(ctx->prop.multiProcessorCount) * 32;
            int64_t rpc = (rows + want - 1) / want;
            const int64_t ty = rw.vpr >= 129 ? 1 : (rw.vpr > 64 ? 2 : (rw.vpr > 32 ? 4 : 8));
            const int64_t trip = ty * 4;
            rpc = ((rpc + trip - 1) / trip) * trip;      // whole trips per CTA
            rw.rows_per_cta = (unsigned long long)rpc;
            const int64_t grid = (rows + rpc - 1) / rpc;
            if (p.nd == 2) nk_ew_rows_kernel<T, NIN, F, 1><<<unsigned(grid), block, 0, ctx->stream>>>(out, a, b, p, rw, f);
            else nk_ew_rows_kernel<T, NIN, F, 2><<<unsigned(grid), block, 0, ctx->stream>>>(out, a, b, p, rw, f);
            return nk_after_launch(ctx, "nk_ew_rows_kernel");
        }
    }
    int grid = nk_grid_for(ctx, p.total, block, 16);
    nk_ew_flat_kernel<T, NIN, F><<<grid, block, 0, ctx->stream>>>(out, a, b, p, f);
    return nk_after_launch(ctx, "nk_ew_flat_kernel");
}

template <class T> T* data_of(nk_buf* b) { return reinterpret_cast<T*>(b->ptr); }

inline bool known_op(int op, bool allow_idy, bool allow_both) {
    if (op >= NK_OP_ADD && op <= NK_OP_POW) return true;
    if (op == NK_OP_IDY) return allow_idy;
    if (op == NK_OP_MUL_BOTH) return allow_both;
    return false;
}

}  // namespace nkew
