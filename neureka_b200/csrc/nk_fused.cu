// Fused elementwise expressions, compiled at run time (NVRTC) -- the CUDA counterpart of the kernels the reference
// generates for `Device.optimizedOperationOf(Function, name)` (devices/Device.java:216-241, model:
// src/main/java/neureka/devices/opencl/utility/CLFunctionCompiler.java:47-196), with one addition the reference's compiler lacks: operands
// broadcast, so `tanh(i0*i1+i1)` over a [4096,1,1024] and a [1,2048,1024] tensor is one pass that reads 24 MiB and
// writes the result once instead of three passes over 32 GiB intermediates.
//
// The host hands over one C expression over x0..x5 built from op_add/op_sub/op_mul/op_div/op_mod/op_pow, f_<id>,
// df_<id> (the 23 scalar functions and their derivatives) and T(<constant>). The generated translation unit embeds the
// very header the op-by-op kernels are compiled from and is compiled without multiply-add contraction, every
// operator rounds to the tensor's type like the separate kernels do, so the fused result equals the op-by-op
// result bit for bit.
//
// NVRTC is looked up with dlopen at the first compilation (no link-time dependency); the compiled image is loaded
// with the runtime's library API. A failure to find or run the compiler is reported, nothing falls back.
#include "nk_internal.h"

#include <dlfcn.h>

#include <cstring>
#include <string>
#include <vector>

// nk_scalarfun.cuh and the nk_op / nk_fun enums as one string (written by build.py next to the objects)
static const char* const k_prelude =
#include "nk_fused_prelude.inc"
    ;

#define NK_FUSED_MAX_IN 6
#define NK_FUSED_MAX_LEAVES 8

// Forward, "rows" form: every tensor has stride 1 or 0 along the innermost merged dim and there are one or two outer dims.
struct FusedRows {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    long long b0, b[NK_FUSED_MAX_IN];
    long long s0[2];                       // drain strides of the outer dims ([1] is the faster one)
    long long s[NK_FUSED_MAX_IN][2];
    unsigned long long rows, rows_per_cta;
    unsigned ext1;                         // extent of the faster outer dim (1 when there is only one)
    unsigned vpr;                          // 128-bit vectors per row
    unsigned stream_mask;                  // bit j: input j runs along the row (stride 1), else one value per row
    unsigned n_outer;
};

// Forward, any view: per-element decode over the merged dims.
struct FusedFlat {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    long long b0, b[NK_FUSED_MAX_IN];
    long long total;
    int nd;
    long long div[NK_MAX_RANK], s0[NK_MAX_RANK], s[NK_FUSED_MAX_IN][NK_MAX_RANK];
};

// Backward: one thread per vector of target elements; sums over the dims the target is broadcast along.
struct FusedGrad {
    void* out;
    const void* err;
    const void* in[NK_FUSED_MAX_IN];
    long long total;                       // target elements / vec
    int nk, nr, vec;                       // kept dims (innermost last), reduced dims (lowest first = fastest), lanes per thread
    unsigned stream_mask;                  // bit j: input j has stride 1 along the innermost kept dim; bit 6: the error
    unsigned invariant_mask;               // bit j: input j does not move along any reduced dim (loaded once); bit 6: the error
    long long kdiv[NK_MAX_RANK], ks0[NK_MAX_RANK], kse[NK_MAX_RANK], ks[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long rext[NK_MAX_RANK], rse[NK_MAX_RANK], rs[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long b0, be, b[NK_FUSED_MAX_IN];
};

struct nk_fused {
    cudaLibrary_t lib = nullptr;
    cudaKernel_t kernel = nullptr;        // forward: flat form; backward: the gradient kernel
    cudaKernel_t rows1 = nullptr, rows2 = nullptr;   // forward, rows form with one / two outer dims
    int grad_target = -1;                 // >= 0: a backward operation for this input
    int n_leaves = 0;
    int dtype = NK_F32;
    int n_in = 0;
    int device = 0;
    uint32_t magic = 0x4e4b4655;  // 'NKFU'
};

namespace {

// ---- NVRTC through dlopen ---------------------------------------------------------------------------------
typedef struct _nvrtcProgram* nvrtcProgram;
struct Nvrtc {
    void* handle = nullptr;
    int (*CreateProgram)(nvrtcProgram*, const char*, const char*, int, const char* const*, const char* const*) = nullptr;
    int (*CompileProgram)(nvrtcProgram, int, const char* const*) = nullptr;
    int (*GetProgramLogSize)(nvrtcProgram, size_t*) = nullptr;
    int (*GetProgramLog)(nvrtcProgram, char*) = nullptr;
    int (*GetCUBINSize)(nvrtcProgram, size_t*) = nullptr;
    int (*GetCUBIN)(nvrtcProgram, char*) = nullptr;
    int (*DestroyProgram)(nvrtcProgram*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    std::string error;
};

Nvrtc* nvrtc() {
    static Nvrtc n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* names[] = {"libnvrtc.so.12", "libnvrtc.so", "/usr/local/cuda/lib64/libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so"};
        for (const char* name : names) {
            n.handle = dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (n.handle) break;
        }
        if (!n.handle) { n.error = std::string("libnvrtc.so.12 not found: ") + (dlerror() ? dlerror() : "?"); return; }
#define NK_SYM(field, sym)                                                                   \
    n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, sym));                     \
    if (!n.field && n.error.empty()) n.error = std::string("libnvrtc lacks ") + sym;
        NK_SYM(CreateProgram, "nvrtcCreateProgram");
        NK_SYM(CompileProgram, "nvrtcCompileProgram");
        NK_SYM(GetProgramLogSize, "nvrtcGetProgramLogSize");
        NK_SYM(GetProgramLog, "nvrtcGetProgramLog");
        NK_SYM(GetCUBINSize, "nvrtcGetCUBINSize");
        NK_SYM(GetCUBIN, "nvrtcGetCUBIN");
        NK_SYM(DestroyProgram, "nvrtcDestroyProgram");
        NK_SYM(GetErrorString, "nvrtcGetErrorString");
#undef NK_SYM
    });
    return &n;
}

// ---- the generated translation unit ---------------------------------------------------------------------------
const char* const k_common_src = R"NKSRC(
#define NK_MAX_RANK 8
#define NK_FUSED_MAX_IN 6
// operators: one rounding to T each, exactly like the separate kernels (this unit is compiled with --fmad=false)
__device__ __forceinline__ T op_add(T a, T b) { return a + b; }
__device__ __forceinline__ T op_sub(T a, T b) { return a - b; }
__device__ __forceinline__ T op_mul(T a, T b) { return a * b; }
__device__ __forceinline__ T op_div(T a, T b) { return a / b; }
__device__ __forceinline__ T op_mod(T a, T b) { return nkf::mod(a, b); }
__device__ __forceinline__ T op_pow(T a, T b) { return nkf::bin<1>(NK_OP_POW, -1, a, b); }
// local derivatives of the operators w.r.t. operand d (the same-shape family's formulas)
__device__ __forceinline__ T dop_div(int d, T a, T b) { return nkf::bin<1>(NK_OP_DIV, d, a, b); }
__device__ __forceinline__ T dop_mod(int d, T a, T b) { return nkf::bin<1>(NK_OP_MOD, d, a, b); }
__device__ __forceinline__ T dop_pow(int d, T a, T b) { return nkf::bin<1>(NK_OP_POW, d, a, b); }
#define NK_F(name, ID)                                                                      \
    __device__ __forceinline__ T f_##name(T a) { return nkf::fun(ID, false, a); }           \
    __device__ __forceinline__ T df_##name(T a) { return nkf::fun(ID, true, a); }
NK_F(abs, NK_FUN_ABS) NK_F(cbrt, NK_FUN_CBRT) NK_F(cos, NK_FUN_COS) NK_F(exp, NK_FUN_EXP) NK_F(gasu, NK_FUN_GASU)
NK_F(gatu, NK_FUN_GATU) NK_F(gaus, NK_FUN_GAUS) NK_F(fast_gaus, NK_FUN_FAST_GAUS) NK_F(gelu, NK_FUN_GELU) NK_F(idy, NK_FUN_IDY)
NK_F(log10, NK_FUN_LOG10) NK_F(ln, NK_FUN_LN) NK_F(quad, NK_FUN_QUAD) NK_F(relu, NK_FUN_RELU) NK_F(selu, NK_FUN_SELU)
NK_F(silu, NK_FUN_SILU) NK_F(sig, NK_FUN_SIG) NK_F(sin, NK_FUN_SIN) NK_F(softplus, NK_FUN_SOFTPLUS)
NK_F(softsign, NK_FUN_SOFTSIGN) NK_F(sqrt, NK_FUN_SQRT) NK_F(tanh, NK_FUN_TANH) NK_F(fast_tanh, NK_FUN_FAST_TANH)
)NKSRC";

const char* const k_forward_src = R"NKSRC(
struct FusedRows {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    long long b0, b[NK_FUSED_MAX_IN];
    long long s0[2];
    long long s[NK_FUSED_MAX_IN][2];
    unsigned long long rows, rows_per_cta;
    unsigned ext1, vpr, stream_mask, n_outer;
};
struct FusedFlat {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    long long b0, b[NK_FUSED_MAX_IN];
    long long total;
    int nd;
    long long div[NK_MAX_RANK], s0[NK_MAX_RANK], s[NK_FUSED_MAX_IN][NK_MAX_RANK];
};

__device__ __forceinline__ T nk_expr(T x0, T x1, T x2, T x3, T x4, T x5) { return NK_EXPR; }
__device__ __forceinline__ T nk_eval(const T* x) {
    return nk_expr(x[0], NK_NIN > 1 ? x[NK_NIN > 1 ? 1 : 0] : T(0), NK_NIN > 2 ? x[NK_NIN > 2 ? 2 : 0] : T(0), NK_NIN > 3 ? x[NK_NIN > 3 ? 3 : 0] : T(0),
                   NK_NIN > 4 ? x[NK_NIN > 4 ? 4 : 0] : T(0), NK_NIN > 5 ? x[NK_NIN > 5 ? 5 : 0] : T(0));
}
// The same expression with the straight-line F32 tanh (nkf::tanh32_fast): inputs that form is not valid for are reported
// through nk_rare instead of branching, so that the elements of a vector are evaluated side by side; the rows kernel
// repeats a vector with the exact form above if any of its elements reported. Without a tanh, or in F64, nk_rare stays
// false and the two forms are the same code.
__device__ __forceinline__ double nk_tanh_flagged(double a, bool&) { return nkf::fun(NK_FUN_TANH, false, a); }
__device__ __forceinline__ float nk_tanh_flagged(float a, bool& rare) { rare = rare || nkf::tanh32_rare(a); return nkf::tanh32_fast(a); }
#define f_tanh(a) nk_tanh_flagged((a), nk_rare)
__device__ __forceinline__ T nk_expr_fast(T x0, T x1, T x2, T x3, T x4, T x5, bool& nk_rare) { return NK_EXPR; }
#undef f_tanh
__device__ __forceinline__ T nk_eval_fast(const T* x, bool& rare) {
    return nk_expr_fast(x[0], NK_NIN > 1 ? x[NK_NIN > 1 ? 1 : 0] : T(0), NK_NIN > 2 ? x[NK_NIN > 2 ? 2 : 0] : T(0), NK_NIN > 3 ? x[NK_NIN > 3 ? 3 : 0] : T(0),
                        NK_NIN > 4 ? x[NK_NIN > 4 ? 4 : 0] : T(0), NK_NIN > 5 ? x[NK_NIN > 5 ? 5 : 0] : T(0), rare);
}

// Rows form. Rows are dealt to CTAs in contiguous blocks; a CTA decodes its first row with one division and then walks
// row by row with an odometer over the (one or two) outer dims -- adds and compares only. Within a row the threads
// stream 128-bit vectors; RPT rows are in flight per thread before the first store.
#define NK_RPT (NK_NIN <= 2 ? 4 : 2)
template <int N_OUTER>
__device__ __forceinline__ void nk_fused_rows(const FusedRows& a) {
    T* __restrict__ out = reinterpret_cast<T*>(a.out);
    const unsigned TX = a.vpr > 128 ? 256u : (a.vpr > 64 ? 128u : (a.vpr > 32 ? 64u : 32u));
    const unsigned TY = 256u / TX;
    const unsigned tx = threadIdx.x % TX, ty = threadIdx.x / TX;
    const unsigned long long r_begin = (unsigned long long)blockIdx.x * a.rows_per_cta;
    unsigned long long r_end = r_begin + a.rows_per_cta;
    if (r_end > a.rows) r_end = a.rows;
    if (r_begin >= r_end) return;
    unsigned long long r = r_begin + ty;
    unsigned i0, i1;
    if (N_OUTER == 2) { i0 = unsigned(r / a.ext1); i1 = unsigned(r - (unsigned long long)i0 * a.ext1); }
    else { i0 = unsigned(r); i1 = 0; }
    long long o0 = a.b0 + (long long)i0 * a.s0[0];
    long long oi[NK_NIN], st[NK_NIN], w[NK_NIN];
    if (N_OUTER == 2) o0 += (long long)i1 * a.s0[1];
#pragma unroll
    for (int j = 0; j < NK_NIN; j++) {
        oi[j] = a.b[j] + (long long)i0 * a.s[j][0] + (N_OUTER == 2 ? (long long)i1 * a.s[j][1] : 0);
        st[j] = (long long)TY * a.s[j][N_OUTER - 1];
        w[j] = N_OUTER == 2 ? a.s[j][0] - (long long)a.ext1 * a.s[j][1] : 0;
    }
    const long long st0 = (long long)TY * a.s0[N_OUTER - 1];
    const long long w0 = N_OUTER == 2 ? a.s0[0] - (long long)a.ext1 * a.s0[1] : 0;
    while (r < r_end) {
        long long q0[NK_RPT], qi[NK_RPT][NK_NIN];
        bool ok[NK_RPT];
#pragma unroll
        for (int u = 0; u < NK_RPT; u++) {
            ok[u] = r < r_end;
            q0[u] = o0;
#pragma unroll
            for (int j = 0; j < NK_NIN; j++) qi[u][j] = oi[j];
            r += TY;
            o0 += st0;
#pragma unroll
            for (int j = 0; j < NK_NIN; j++) oi[j] += st[j];
            if (N_OUTER == 2) {
                i1 += TY;
                while (i1 >= a.ext1) {   // TY <= 8 < any merged extent
                    i1 -= a.ext1; o0 += w0;
#pragma unroll
                    for (int j = 0; j < NK_NIN; j++) oi[j] += w[j];
                }
            }
        }
        for (unsigned c = tx; c < a.vpr; c += TX) {
            T x[NK_RPT][NK_NIN][VECW];
#pragma unroll
            for (int u = 0; u < NK_RPT; u++) {
                if (!ok[u]) continue;
#pragma unroll
                for (int j = 0; j < NK_NIN; j++) {
                    const T* src = reinterpret_cast<const T*>(a.in[j]) + qi[u][j];
                    if ((a.stream_mask >> j) & 1u) *reinterpret_cast<V*>(x[u][j]) = __ldg(reinterpret_cast<const V*>(src) + c);
                    else { const T v = src[0];
#pragma unroll
                        for (int e = 0; e < VECW; e++) x[u][j][e] = v; }
                }
            }
#pragma unroll
            for (int u = 0; u < NK_RPT; u++) {
                if (!ok[u]) continue;
                T res[VECW];
                bool rare = false;
#pragma unroll
                for (int e = 0; e < VECW; e++) {
                    T in[NK_NIN];
#pragma unroll
                    for (int j = 0; j < NK_NIN; j++) in[j] = x[u][j][e];
                    res[e] = nk_eval_fast(in, rare);
                }
                if (rare) {
#pragma unroll
                    for (int e = 0; e < VECW; e++) {
                        T in[NK_NIN];
#pragma unroll
                        for (int j = 0; j < NK_NIN; j++) in[j] = x[u][j][e];
                        res[e] = nk_eval(in);
                    }
                }
                __stcs(reinterpret_cast<V*>(out + q0[u]) + c, *reinterpret_cast<V*>(res));
            }
        }
    }
}
// NK_MIN_CTAS: 3 for expressions made of operators only -- a pure stream, where three resident CTAs per SM (24 warps' worth of
// loads and stores in flight) matter more than registers; 1 when scalar functions are called (their evaluation wants them).
extern "C" __global__ void __launch_bounds__(256, NK_MIN_CTAS) nk_fused_rows1(const FusedRows a) { nk_fused_rows<1>(a); }
extern "C" __global__ void __launch_bounds__(256, NK_MIN_CTAS) nk_fused_rows2(const FusedRows a) { nk_fused_rows<2>(a); }

extern "C" __global__ void __launch_bounds__(256) nk_fused_kernel(const FusedFlat a) {
    T* out = reinterpret_cast<T*>(a.out);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < a.total; i += stride) {
        long long rem = i, o0 = a.b0, oi[NK_NIN];
#pragma unroll
        for (int j = 0; j < NK_NIN; j++) oi[j] = a.b[j];
        for (int k = 0; k < a.nd; k++) {
            const long long idx = rem / a.div[k];
            rem -= idx * a.div[k];
            o0 += idx * a.s0[k];
#pragma unroll
            for (int j = 0; j < NK_NIN; j++) oi[j] += idx * a.s[j][k];
        }
        T in[NK_NIN];
#pragma unroll
        for (int j = 0; j < NK_NIN; j++) in[j] = reinterpret_cast<const T*>(a.in[j])[oi[j]];
        out[o0] = nk_eval(in);
    }
}
)NKSRC";

// Backward of an elementwise expression w.r.t. one input, with the broadcast dims of that input summed away in the
// same kernel: gradient[idx] = sum over the dims the input is broadcast along of sum over its occurrences in the
// expression of term_l(error, x0 .. x5). The host hands over NK_TERMS, C statements that set term[0 .. NK_NLEAF-1] from
// e and x0..x5 with one rounding per operator like the separate kernels; every occurrence has its own accumulator, the
// reduction runs with the lowest reduced dim fastest (the order of the separate reduction kernels), and the
// accumulators are added in occurrence order at the end.
const char* const k_grad_src = R"NKSRC(
struct FusedGrad {
    void* out;
    const void* err;
    const void* in[NK_FUSED_MAX_IN];
    long long total;
    int nk, nr, vec;
    unsigned stream_mask, invariant_mask;
    long long kdiv[NK_MAX_RANK], ks0[NK_MAX_RANK], kse[NK_MAX_RANK], ks[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long rext[NK_MAX_RANK], rse[NK_MAX_RANK], rs[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long b0, be, b[NK_FUSED_MAX_IN];
};
__device__ __forceinline__ void nk_terms(T e, T x0, T x1, T x2, T x3, T x4, T x5, T* term) { NK_TERMS }

template <int VEC>
__device__ __forceinline__ void nk_grad_body(const FusedGrad& a) {
    T* out = reinterpret_cast<T*>(a.out);
    const T* err = reinterpret_cast<const T*>(a.err);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < a.total; v += stride) {
        long long rem = v * VEC, o0 = a.b0, oe = a.be, oi[NK_NIN];
#pragma unroll
        for (int j = 0; j < NK_NIN; j++) oi[j] = a.b[j];
        for (int k = 0; k < a.nk; k++) {
            const long long idx = rem / a.kdiv[k];
            rem -= idx * a.kdiv[k];
            o0 += idx * a.ks0[k];
            oe += idx * a.kse[k];
#pragma unroll
            for (int j = 0; j < NK_NIN; j++) oi[j] += idx * a.ks[j][k];
        }
        T acc[NK_NLEAF][VEC];
#pragma unroll
        for (int l = 0; l < NK_NLEAF; l++)
#pragma unroll
            for (int e = 0; e < VEC; e++) acc[l][e] = T(0);
        T x[NK_NIN + 1][VEC];   // [NK_NIN] is the error
        auto fetch = [&](int j, const T* p, bool streams) {
            if (VEC > 1 && streams) *reinterpret_cast<V*>(x[j]) = *reinterpret_cast<const V*>(p);
            else { const T s = p[0];
#pragma unroll
                for (int e = 0; e < VEC; e++) x[j][e] = s; }
        };
        // operands that do not move along the reduced dims (the target itself, for one) are read once
#pragma unroll
        for (int j = 0; j < NK_NIN; j++)
            if ((a.invariant_mask >> j) & 1u) fetch(j, reinterpret_cast<const T*>(a.in[j]) + oi[j], (a.stream_mask >> j) & 1u);
        if ((a.invariant_mask >> 6) & 1u) fetch(NK_NIN, err + oe, (a.stream_mask >> 6) & 1u);
        long long q[NK_MAX_RANK];
        for (int k = 0; k < a.nr; k++) q[k] = 0;
        while (true) {
#pragma unroll
            for (int j = 0; j < NK_NIN; j++)
                if (!((a.invariant_mask >> j) & 1u)) fetch(j, reinterpret_cast<const T*>(a.in[j]) + oi[j], (a.stream_mask >> j) & 1u);
            if (!((a.invariant_mask >> 6) & 1u)) fetch(NK_NIN, err + oe, (a.stream_mask >> 6) & 1u);
#pragma unroll
            for (int e = 0; e < VEC; e++) {
                T term[NK_NLEAF];
                nk_terms(x[NK_NIN][e], x[0][e], x[NK_NIN > 1 ? 1 : 0][e], x[NK_NIN > 2 ? 2 : 0][e], x[NK_NIN > 3 ? 3 : 0][e],
                         x[NK_NIN > 4 ? 4 : 0][e], x[NK_NIN > 5 ? 5 : 0][e], term);
#pragma unroll
                for (int l = 0; l < NK_NLEAF; l++) acc[l][e] += term[l];
            }
            int k = 0;
            for (; k < a.nr; k++) {
                q[k]++; oe += a.rse[k];
#pragma unroll
                for (int j = 0; j < NK_NIN; j++) oi[j] += a.rs[j][k];
                if (q[k] < a.rext[k]) break;
                oe -= q[k] * a.rse[k];
#pragma unroll
                for (int j = 0; j < NK_NIN; j++) oi[j] -= q[k] * a.rs[j][k];
                q[k] = 0;
            }
            if (k >= a.nr) break;
        }
        T res[VEC];
#pragma unroll
        for (int e = 0; e < VEC; e++) {
            res[e] = acc[0][e];
#pragma unroll
            for (int l = 1; l < NK_NLEAF; l++) res[e] += acc[l][e];
        }
        if (VEC > 1) *reinterpret_cast<V*>(out + o0) = *reinterpret_cast<V*>(res);
        else out[o0] = res[0];
    }
}
extern "C" __global__ void __launch_bounds__(256) nk_fused_grad_kernel(const FusedGrad a) {
    if (a.vec > 1) nk_grad_body<VECW>(a); else nk_grad_body<1>(a);
}
)NKSRC";

}  // namespace

namespace {

// Compiles one translation unit (prelude + common operators + `body`) for the context's GPU and loads the image.
int compile_unit(nk_ctx* ctx, const char* who, int dtype, int n_inputs, const std::string& defines, const char* body, cudaLibrary_t* lib) {
    Nvrtc* rt = nvrtc();
    if (!rt->error.empty()) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "%s: run-time compiler unavailable (%s)", who, rt->error.c_str());
    std::string src;
    src += dtype == NK_F32 ? "typedef float T;\ntypedef float4 V;\n#define VECW 4\n" : "typedef double T;\ntypedef double2 V;\n#define VECW 2\n";
    src += "#define NK_NIN " + std::to_string(n_inputs) + "\n";
    src += defines;
    src += k_prelude;
    src += k_common_src;
    src += body;

    nvrtcProgram prog = nullptr;
    int rc = rt->CreateProgram(&prog, src.c_str(), "nk_fused.cu", 0, nullptr, nullptr);
    if (rc) return nk_fail(ctx, NK_ERR_CUDA, "nvrtcCreateProgram: %s", rt->GetErrorString(rc));
    char arch[64];
    snprintf(arch, sizeof(arch), "--gpu-architecture=sm_%d%d%s", ctx->prop.major, ctx->prop.minor, ctx->prop.major >= 9 ? "a" : "");
    const char* opts[] = {arch, "--fmad=false", "--std=c++17", "-default-device"};
    rc = rt->CompileProgram(prog, 4, opts);
    if (rc) {
        size_t n = 0;
        rt->GetProgramLogSize(prog, &n);
        std::string log(n ? n : 1, '\0');
        if (n) rt->GetProgramLog(prog, &log[0]);
        rt->DestroyProgram(&prog);
        if (log.size() > 1500) log.resize(1500);
        return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: the expression does not compile (%s): %s", who, rt->GetErrorString(rc), log.c_str());
    }
    size_t n = 0;
    rc = rt->GetCUBINSize(prog, &n);
    std::vector<char> image(n);
    if (!rc && n) rc = rt->GetCUBIN(prog, image.data());
    rt->DestroyProgram(&prog);
    if (rc || !n) return nk_fail(ctx, NK_ERR_CUDA, "%s: no device image (%s)", who, rc ? rt->GetErrorString(rc) : "empty");
    cudaError_t e = cudaLibraryLoadData(lib, image.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaLibraryLoadData (fused kernel)");
    return NK_OK;
}

// Broadcast shapes of a fused call: per dim an operand follows the drain index where it has the drain's extent and
// stays at 0 where its extent is 1 (Broadcast.java:76-95); anything else is a shape error.
int operand_strides(nk_ctx* ctx, const char* who, int rank, const int64_t* full, const NkView& v, int j, int64_t* s) {
    for (int k = 0; k < rank; k++) {
        if (v.shape[k] == full[k]) s[k] = v.estride[k];
        else if (v.shape[k] == 1) s[k] = 0;
        else return nk_fail(ctx, NK_ERR_BAD_ARG, "%s: operand %d has extent %lld in dim %d, the result %lld", who, j, (long long)v.shape[k], k, (long long)full[k]);
    }
    return NK_OK;
}

bool aligned16(const void* base, int64_t elems, int es) { return ((reinterpret_cast<uintptr_t>(base) + size_t(elems) * es) & 15) == 0; }

}  // namespace

extern "C" int nk_fused_compile(nk_ctx* ctx, int32_t dtype, int32_t n_inputs, const char* expr, nk_fused** out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: out pointer is null");
    *out = nullptr;
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_compile: dtype %d not supported (F32/F64 only)", dtype);
    if (n_inputs < 1 || n_inputs > NK_FUSED_MAX_IN) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: 1..%d inputs, got %d", NK_FUSED_MAX_IN, n_inputs);
    if (!expr || !*expr) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: empty expression");
    nk_fused* f = new (std::nothrow) nk_fused();
    if (!f) return nk_fail(ctx, NK_ERR_OOM, "nk_fused_compile: out of host memory");
    const bool calls_functions = strstr(expr, "f_") != nullptr || strstr(expr, "op_pow") != nullptr || strstr(expr, "op_mod") != nullptr;
    const std::string defs = std::string("#define NK_EXPR (") + expr + ")\n#define NK_MIN_CTAS " + (calls_functions ? "1" : "3") + "\n";
    int st = compile_unit(ctx, "nk_fused_compile", dtype, n_inputs, defs, k_forward_src, &f->lib);
    if (st) { delete f; return st; }
    cudaError_t e = cudaLibraryGetKernel(&f->kernel, f->lib, "nk_fused_kernel");
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&f->rows1, f->lib, "nk_fused_rows1");
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&f->rows2, f->lib, "nk_fused_rows2");
    if (e != cudaSuccess) {
        cudaLibraryUnload(f->lib);
        delete f;
        return nk_cuda_fail(ctx, e, "cudaLibraryGetKernel (fused kernel)");
    }
    f->dtype = dtype;
    f->n_in = n_inputs;
    f->device = ctx->device;
    *out = f;
    return NK_OK;
}

extern "C" int nk_fused_compile_grad(nk_ctx* ctx, int32_t dtype, int32_t n_inputs, int32_t target, int32_t n_leaves, const char* terms,
                                     nk_fused** out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile_grad: out pointer is null");
    *out = nullptr;
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_compile_grad: dtype %d not supported (F32/F64 only)", dtype);
    if (n_inputs < 1 || n_inputs > NK_FUSED_MAX_IN) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile_grad: 1..%d inputs, got %d", NK_FUSED_MAX_IN, n_inputs);
    if (target < 0 || target >= n_inputs) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile_grad: target %d is not one of the %d inputs", target, n_inputs);
    if (n_leaves < 1 || n_leaves > NK_FUSED_MAX_LEAVES)
        return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_compile_grad: 1..%d occurrences of the target, got %d", NK_FUSED_MAX_LEAVES, n_leaves);
    if (!terms || !*terms) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile_grad: empty statement list");
    nk_fused* f = new (std::nothrow) nk_fused();
    if (!f) return nk_fail(ctx, NK_ERR_OOM, "nk_fused_compile_grad: out of host memory");
    std::string defs = "#define NK_NLEAF " + std::to_string(n_leaves) + "\n#define NK_TERMS " + terms + "\n";
    int st = compile_unit(ctx, "nk_fused_compile_grad", dtype, n_inputs, defs, k_grad_src, &f->lib);
    if (st) { delete f; return st; }
    cudaError_t e = cudaLibraryGetKernel(&f->kernel, f->lib, "nk_fused_grad_kernel");
    if (e != cudaSuccess) {
        cudaLibraryUnload(f->lib);
        delete f;
        return nk_cuda_fail(ctx, e, "cudaLibraryGetKernel (fused gradient kernel)");
    }
    f->dtype = dtype;
    f->n_in = n_inputs;
    f->device = ctx->device;
    f->grad_target = target;
    f->n_leaves = n_leaves;
    *out = f;
    return NK_OK;
}

extern "C" int nk_fused_run(nk_ctx* ctx, nk_fused* f, int32_t rank, nk_buf* drn, const int32_t* cfg0, nk_buf* const* srcs, const int32_t* const* cfgs) {
    NK_CHECK_CTX(ctx);
    if (!f || f->magic != 0x4e4b4655 || f->grad_target >= 0) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: not a fused forward operation");
    if (f->device != ctx->device) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: compiled for device %d, called on device %d", f->device, ctx->device);
    if (!srcs || !cfgs) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: null operand list");
    NkView v0, v[NK_FUSED_MAX_IN];
    int st;
    if ((st = nk_view_parse(ctx, "nk_fused_run(drain)", drn, cfg0, rank, f->dtype, &v0))) return st;
    for (int j = 0; j < f->n_in; j++)
        if ((st = nk_view_parse(ctx, "nk_fused_run(src)", srcs[j], cfgs[j], rank, f->dtype, &v[j]))) return st;
    if (!v0.imap_row_major)
        return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_run: the drain must be indexed row-major (a fresh output tensor is)");
    int64_t s[NK_FUSED_MAX_IN][NK_MAX_RANK];
    for (int j = 0; j < f->n_in; j++)
        if ((st = operand_strides(ctx, "nk_fused_run", rank, v0.shape, v[j], j, s[j]))) return st;
    // drop size-1 dims, merge neighbours across which every tensor is linear
    int64_t ext[NK_MAX_RANK], m0[NK_MAX_RANK], m[NK_FUSED_MAX_IN][NK_MAX_RANK];
    int nd = 0;
    for (int k = 0; k < rank; k++) {
        const int64_t e = v0.shape[k];
        if (e == 1) continue;
        bool merge = nd > 0 && m0[nd - 1] == e * v0.estride[k];
        for (int j = 0; j < f->n_in && merge; j++) merge = m[j][nd - 1] == e * s[j][k];
        if (merge) {
            ext[nd - 1] *= e;
            m0[nd - 1] = v0.estride[k];
            for (int j = 0; j < f->n_in; j++) m[j][nd - 1] = s[j][k];
        } else {
            ext[nd] = e;
            m0[nd] = v0.estride[k];
            for (int j = 0; j < f->n_in; j++) m[j][nd] = s[j][k];
            nd++;
        }
    }
    if (nd == 0) { ext[0] = 1; m0[0] = 1; for (int j = 0; j < f->n_in; j++) m[j][0] = 0; nd = 1; }
    // a fully linear problem is one long row: cut it into rows of 1024 so that it takes the rows form as well
    if (nd == 1 && ext[0] >= 8192 && ext[0] % 1024 == 0) {
        ext[1] = 1024; m0[1] = m0[0];
        for (int j = 0; j < f->n_in; j++) m[j][1] = m[j][0];
        ext[0] /= 1024; m0[0] *= 1024;
        for (int j = 0; j < f->n_in; j++) m[j][0] *= 1024;
        nd = 2;
    }
    const int es = int(nk_dtype_size(f->dtype)), W = 16 / es;
    const int last = nd - 1;
    // ---- rows form: long unit-stride rows, one or two outer dims, everything 16-byte aligned ----
    bool rows_ok = (nd == 2 || nd == 3) && m0[last] == 1 && ext[last] >= 64 && ext[last] % W == 0 && ext[last] / W < (int64_t(1) << 31) &&
                   aligned16(drn->ptr, v0.base, es) && (nd == 2 || ext[1] >= 8);
    unsigned stream_mask = 0;
    for (int j = 0; j < f->n_in && rows_ok; j++) {
        if (m[j][last] == 1) { stream_mask |= 1u << j; rows_ok = aligned16(srcs[j]->ptr, v[j].base, es); }
        else if (m[j][last] != 0) rows_ok = false;
    }
    for (int k = 0; k < last && rows_ok; k++) {
        rows_ok = m0[k] % W == 0 && ext[k] < (int64_t(1) << 31);
        for (int j = 0; j < f->n_in && rows_ok; j++)
            if ((stream_mask >> j) & 1u) rows_ok = m[j][k] % W == 0;
    }
    if (rows_ok) {
        FusedRows a;
        memset(&a, 0, sizeof(a));
        a.out = drn->ptr;
        a.b0 = v0.base;
        a.n_outer = unsigned(nd - 1);
        a.ext1 = nd == 3 ? unsigned(ext[1]) : 1u;
        a.vpr = unsigned(ext[last] / W);
        a.stream_mask = stream_mask;
        int64_t rows = 1;
        for (int k = 0; k < last; k++) { rows *= ext[k]; a.s0[k] = m0[k]; }
        for (int j = 0; j < f->n_in; j++) {
            a.in[j] = srcs[j]->ptr;
            a.b[j] = v[j].base;
            for (int k = 0; k < last; k++) a.s[j][k] = m[j][k];
        }
        a.rows = (unsigned long long)rows;
        // enough CTAs to fill the machine several times over, each with a contiguous block of rows, whole trips per CTA
        const int64_t want = int64_t(ctx->prop.multiProcessorCount) * 32;
        int64_t rpc = (rows + want - 1) / want;
        const int64_t ty = a.vpr > 128 ? 1 : (a.vpr > 64 ? 2 : (a.vpr > 32 ? 4 : 8));
        const int64_t trip = ty * (f->n_in <= 2 ? 4 : 2);
        rpc = ((rpc + trip - 1) / trip) * trip;
        a.rows_per_cta = (unsigned long long)rpc;
        const int64_t grid = (rows + rpc - 1) / rpc;
        void* params[] = {&a};
        NK_CUDA(ctx, cudaLaunchKernel(reinterpret_cast<const void*>(nd == 2 ? f->rows1 : f->rows2), dim3(unsigned(grid)), dim3(256), params, 0, ctx->stream));
        return nk_after_launch(ctx, "nk_fused_rows_kernel");
    }
    // ---- any other view: per-element decode ----
    FusedFlat a;
    memset(&a, 0, sizeof(a));
    a.out = drn->ptr;
    a.b0 = v0.base;
    a.nd = nd;
    a.total = 1;
    for (int k = nd - 1; k >= 0; k--) { a.div[k] = a.total; a.total *= ext[k]; a.s0[k] = m0[k]; }
    for (int j = 0; j < f->n_in; j++) {
        a.in[j] = srcs[j]->ptr;
        a.b[j] = v[j].base;
        for (int k = 0; k < nd; k++) a.s[j][k] = m[j][k];
    }
    if (a.total == 0) return NK_OK;
    void* params[] = {&a};
    NK_CUDA(ctx, cudaLaunchKernel(reinterpret_cast<const void*>(f->kernel), dim3(unsigned(nk_grid_for(ctx, a.total, 256, 16))), dim3(256), params, 0, ctx->stream));
    return nk_after_launch(ctx, "nk_fused_kernel");
}

extern "C" int nk_fused_run_grad(nk_ctx* ctx, nk_fused* f, int32_t rank, nk_buf* grad, const int32_t* cfg_grad, nk_buf* err, const int32_t* cfg_err,
                                 nk_buf* const* srcs, const int32_t* const* cfgs) {
    NK_CHECK_CTX(ctx);
    if (!f || f->magic != 0x4e4b4655 || f->grad_target < 0) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run_grad: not a fused backward operation");
    if (f->device != ctx->device) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run_grad: compiled for device %d, called on device %d", f->device, ctx->device);
    if (!srcs || !cfgs) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run_grad: null operand list");
    NkView vg, ve, v[NK_FUSED_MAX_IN];
    int st;
    if ((st = nk_view_parse(ctx, "nk_fused_run_grad(gradient)", grad, cfg_grad, rank, f->dtype, &vg))) return st;
    if ((st = nk_view_parse(ctx, "nk_fused_run_grad(error)", err, cfg_err, rank, f->dtype, &ve))) return st;
    for (int j = 0; j < f->n_in; j++)
        if ((st = nk_view_parse(ctx, "nk_fused_run_grad(src)", srcs[j], cfgs[j], rank, f->dtype, &v[j]))) return st;
    if (!vg.imap_row_major) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_run_grad: the gradient must be indexed row-major");
    // the full index space: per dim the largest extent among the operands (the forward result's shape)
    int64_t full[NK_MAX_RANK];
    for (int k = 0; k < rank; k++) {
        full[k] = 1;
        for (int j = 0; j < f->n_in; j++) full[k] = v[j].shape[k] > full[k] ? v[j].shape[k] : full[k];
    }
    const NkView& vt = v[f->grad_target];
    for (int k = 0; k < rank; k++)
        if (vg.shape[k] != vt.shape[k])
            return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run_grad: gradient extent %lld in dim %d, its input has %lld", (long long)vg.shape[k], k, (long long)vt.shape[k]);
    int64_t s[NK_FUSED_MAX_IN][NK_MAX_RANK], se[NK_MAX_RANK];
    for (int j = 0; j < f->n_in; j++)
        if ((st = operand_strides(ctx, "nk_fused_run_grad", rank, full, v[j], j, s[j]))) return st;
    if ((st = operand_strides(ctx, "nk_fused_run_grad(error)", rank, full, ve, -1, se))) return st;   // the error: result-shaped, or one value broadcast
    FusedGrad a;
    memset(&a, 0, sizeof(a));
    a.out = grad->ptr;
    a.err = err->ptr;
    a.b0 = vg.base; a.be = ve.base;
    a.invariant_mask = 0x7f;
    for (int j = 0; j < f->n_in; j++) { a.in[j] = srcs[j]->ptr; a.b[j] = v[j].base; }
    int64_t total = 1;
    int innermost_kept = -1;
    for (int k = 0; k < rank; k++) {
        if (full[k] == 1) continue;
        if (vt.shape[k] == full[k]) {   // kept: part of the gradient's own index
            const int n = a.nk++;
            a.kdiv[n] = full[k];        // extents for now, divisors below
            a.ks0[n] = vg.estride[k];
            a.kse[n] = se[k];
            for (int j = 0; j < f->n_in; j++) a.ks[j][n] = s[j][k];
            total *= full[k];
            innermost_kept = k;
        } else {                        // the target is broadcast here: summed away
            const int n = a.nr++;
            a.rext[n] = full[k];
            a.rse[n] = se[k];
            if (se[k] != 0) a.invariant_mask &= ~(1u << 6);
            for (int j = 0; j < f->n_in; j++) {
                a.rs[j][n] = s[j][k];
                if (s[j][k] != 0) a.invariant_mask &= ~(1u << j);
            }
        }
    }
    // 128-bit lanes along the innermost kept dim when it is the innermost dim of the whole index space and every
    // tensor is unit-stride or broadcast along it
    const int es = int(nk_dtype_size(f->dtype)), W = 16 / es;
    int last_full = -1;
    for (int k = 0; k < rank; k++) if (full[k] != 1) last_full = k;
    bool vec = a.nk > 0 && innermost_kept == last_full && vg.estride[innermost_kept] == 1 && full[innermost_kept] % W == 0 &&
               aligned16(grad->ptr, vg.base, es);
    if (vec) {
        const int n = a.nk - 1;
        auto lane_ok = [&](long long stride, const void* ptr, int64_t base, const long long* ks, const long long* rs, unsigned bit) {
            if (stride == 0) return true;
            if (stride != 1 || !aligned16(ptr, base, es)) return false;
            for (int q = 0; q < n; q++) if (ks[q] % W) return false;
            for (int q = 0; q < a.nr; q++) if (rs[q] % W) return false;
            a.stream_mask |= bit;
            return true;
        };
        vec = lane_ok(a.kse[n], err->ptr, ve.base, a.kse, a.rse, 1u << 6);
        for (int j = 0; j < f->n_in && vec; j++) vec = lane_ok(a.ks[j][n], srcs[j]->ptr, v[j].base, a.ks[j], a.rs[j], 1u << j);
        for (int q = 0; q < n && vec; q++) vec = a.ks0[q] % W == 0;
    }
    if (!vec) a.stream_mask = 0;
    a.vec = vec ? W : 1;
    int64_t d = 1;
    for (int n = a.nk - 1; n >= 0; n--) { const int64_t e = a.kdiv[n]; a.kdiv[n] = d; d *= e; }
    a.total = total / a.vec;
    if (a.total == 0) return NK_OK;
    void* params[] = {&a};
    NK_CUDA(ctx, cudaLaunchKernel(reinterpret_cast<const void*>(f->kernel), dim3(unsigned(nk_grid_for(ctx, a.total, 256, 8))), dim3(256), params, 0, ctx->stream));
    return nk_after_launch(ctx, "nk_fused_grad_kernel");
}

extern "C" int nk_fused_free(nk_fused* f) {
    if (!f || f->magic != 0x4e4b4655) return NK_ERR_BAD_ARG;
    cudaSetDevice(f->device);
    if (f->lib) cudaLibraryUnload(f->lib);
    f->magic = 0;
    delete f;
    return NK_OK;
}
