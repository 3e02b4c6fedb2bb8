// Fused elementwise expressions, compiled at run time (NVRTC) -- the CUDA counterpart of the kernels the reference
// generates for `Device.optimizedOperationOf(Function, name)` (devices/Device.java:216-241, model:
// backend/ocl/utility/CLFunctionCompiler.java:47-196), with one addition the reference's compiler lacks: operands
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

#include <string>
#include <vector>

// nk_scalarfun.cuh and the nk_op / nk_fun enums as one string (written by build.py next to the objects)
static const char* const k_prelude =
#include "nk_fused_prelude.inc"
    ;

#define NK_FUSED_MAX_IN 6

struct FusedPlan {
    int nd;                       // merged dims, innermost last
    int vec;                      // elements per work item along the innermost dim (4 or 1)
    int n_in;
    int wide;                     // unit index needs 64 bits
    long long units;              // row groups * chunks per row
    long long chunks;             // work-item groups per row
    long long inner;              // innermost extent
    long long rows;               // product of the outer extents
    long long ext[NK_MAX_RANK];
    long long s0[NK_MAX_RANK];
    long long s[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long b0, b[NK_FUSED_MAX_IN];
};

struct FusedArgs {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    FusedPlan p;
};

struct nk_fused {
    cudaLibrary_t lib = nullptr;
    cudaKernel_t kernel = nullptr;
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
const char* const k_kernel_src = R"NKSRC(
#define NK_MAX_RANK 8
#define NK_FUSED_MAX_IN 6
struct FusedPlan {
    int nd, vec, n_in, wide;
    long long units, chunks, inner, rows;
    long long ext[NK_MAX_RANK];
    long long s0[NK_MAX_RANK];
    long long s[NK_FUSED_MAX_IN][NK_MAX_RANK];
    long long b0, b[NK_FUSED_MAX_IN];
};
struct FusedArgs {
    void* out;
    const void* in[NK_FUSED_MAX_IN];
    FusedPlan p;
};

// operators: one rounding to T each, exactly like the separate kernels (this unit is compiled with --fmad=false)
__device__ __forceinline__ T op_add(T a, T b) { return a + b; }
__device__ __forceinline__ T op_sub(T a, T b) { return a - b; }
__device__ __forceinline__ T op_mul(T a, T b) { return a * b; }
__device__ __forceinline__ T op_div(T a, T b) { return a / b; }
__device__ __forceinline__ T op_mod(T a, T b) { return nkf::mod(a, b); }
__device__ __forceinline__ T op_pow(T a, T b) { return nkf::bin<1>(NK_OP_POW, -1, a, b); }
#define NK_F(name, ID)                                                                      \
    __device__ __forceinline__ T f_##name(T a) { return nkf::fun(ID, false, a); }           \
    __device__ __forceinline__ T df_##name(T a) { return nkf::fun(ID, true, a); }
NK_F(abs, NK_FUN_ABS) NK_F(cbrt, NK_FUN_CBRT) NK_F(cos, NK_FUN_COS) NK_F(exp, NK_FUN_EXP) NK_F(gasu, NK_FUN_GASU)
NK_F(gatu, NK_FUN_GATU) NK_F(gaus, NK_FUN_GAUS) NK_F(fast_gaus, NK_FUN_FAST_GAUS) NK_F(gelu, NK_FUN_GELU) NK_F(idy, NK_FUN_IDY)
NK_F(log10, NK_FUN_LOG10) NK_F(ln, NK_FUN_LN) NK_F(quad, NK_FUN_QUAD) NK_F(relu, NK_FUN_RELU) NK_F(selu, NK_FUN_SELU)
NK_F(silu, NK_FUN_SILU) NK_F(sig, NK_FUN_SIG) NK_F(sin, NK_FUN_SIN) NK_F(softplus, NK_FUN_SOFTPLUS)
NK_F(softsign, NK_FUN_SOFTSIGN) NK_F(sqrt, NK_FUN_SQRT) NK_F(tanh, NK_FUN_TANH) NK_F(fast_tanh, NK_FUN_FAST_TANH)

__device__ __forceinline__ T nk_expr(T x0, T x1, T x2, T x3, T x4, T x5) { return NK_EXPR; }

// A work unit is one chunk (256 threads x VEC elements) of a group of NK_ROWS consecutive rows of the merged index
// space: the first row is decoded with divisions (32-bit unless the problem needs more), the others follow by counting
// the row index up with carry; all loads of the group are issued before the first result is computed, so a thread
// keeps NK_ROWS x NK_NIN 128-bit loads in flight.
#define NK_ROWS 2
template <int VEC, class IDX>
__device__ __forceinline__ void nk_fused_body(const FusedArgs& a) {
    const FusedPlan& p = a.p;
    T* out = reinterpret_cast<T*>(a.out);
    const int last = p.nd - 1;
    for (IDX unit = blockIdx.x; unit < IDX(p.units); unit += gridDim.x) {
        const IDX grp = unit / IDX(p.chunks);
        const long long col = (long long)(unit - grp * IDX(p.chunks)) * (256 * VEC) + threadIdx.x * VEC;
        if (col >= p.inner) continue;
        // ---- first row of the group: digits by division ----
        long long idx[NK_MAX_RANK - 1];
        long long o0 = p.b0 + col * p.s0[last];
        long long oi[NK_NIN];
#pragma unroll
        for (int j = 0; j < NK_NIN; j++) oi[j] = p.b[j] + col * p.s[j][last];
        {
            IDX row = grp * NK_ROWS;
#pragma unroll
            for (int k = NK_MAX_RANK - 2; k >= 0; k--) {
                if (k < last) {
                    const IDX q = row / IDX(p.ext[k]);
                    idx[k] = (long long)(row - q * IDX(p.ext[k]));
                    row = q;
                    o0 += idx[k] * p.s0[k];
#pragma unroll
                    for (int j = 0; j < NK_NIN; j++) oi[j] += idx[k] * p.s[j][k];
                } else {
                    idx[k] = 0;
                }
            }
        }
        const long long rows_left = p.rows - (long long)grp * NK_ROWS;
        long long ro[NK_ROWS], ri[NK_ROWS][NK_NIN];
#pragma unroll
        for (int r = 0; r < NK_ROWS; r++) {
            ro[r] = o0;
#pragma unroll
            for (int j = 0; j < NK_NIN; j++) ri[r][j] = oi[j];
            // next row: count up, innermost outer dim first
            bool carry = true;
#pragma unroll
            for (int k = NK_MAX_RANK - 2; k >= 0; k--) {
                if (k < last && carry) {
                    idx[k]++;
                    o0 += p.s0[k];
#pragma unroll
                    for (int j = 0; j < NK_NIN; j++) oi[j] += p.s[j][k];
                    if (idx[k] < p.ext[k]) {
                        carry = false;
                    } else {
                        idx[k] = 0;
                        o0 -= p.ext[k] * p.s0[k];
#pragma unroll
                        for (int j = 0; j < NK_NIN; j++) oi[j] -= p.ext[k] * p.s[j][k];
                    }
                }
            }
        }
        T x[NK_ROWS][NK_NIN][VEC];
#pragma unroll
        for (int r = 0; r < NK_ROWS; r++) {
            if (r < rows_left) {
#pragma unroll
                for (int j = 0; j < NK_NIN; j++) {
                    const T* src = reinterpret_cast<const T*>(a.in[j]) + ri[r][j];
                    if (VEC == 1) {
                        x[r][j][0] = src[0];
                    } else if (p.s[j][last] == 0) {
                        const T v = src[0];
#pragma unroll
                        for (int e = 0; e < VEC; e++) x[r][j][e] = v;
                    } else {
                        *reinterpret_cast<V*>(x[r][j]) = *reinterpret_cast<const V*>(src);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < NK_ROWS; r++) {
            if (r < rows_left) {
                T res[VEC];
#pragma unroll
                for (int e = 0; e < VEC; e++) {
                    T in[6];
#pragma unroll
                    for (int j = 0; j < 6; j++) in[j] = j < NK_NIN ? x[r][j < NK_NIN ? j : 0][e] : T(0);
                    res[e] = nk_expr(in[0], in[1], in[2], in[3], in[4], in[5]);
                }
                if (VEC == 1) out[ro[r]] = res[0];
                else *reinterpret_cast<V*>(out + ro[r]) = *reinterpret_cast<V*>(res);
            }
        }
    }
}

extern "C" __global__ void __launch_bounds__(256, 4) nk_fused_kernel(const FusedArgs a) {
    if (a.p.vec > 1) {
        if (a.p.wide) nk_fused_body<VECW, long long>(a); else nk_fused_body<VECW, unsigned>(a);
    } else {
        if (a.p.wide) nk_fused_body<1, long long>(a); else nk_fused_body<1, unsigned>(a);
    }
}
)NKSRC";

}  // namespace

extern "C" int nk_fused_compile(nk_ctx* ctx, int32_t dtype, int32_t n_inputs, const char* expr, nk_fused** out) {
    NK_CHECK_CTX(ctx);
    if (!out) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: out pointer is null");
    *out = nullptr;
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_compile: dtype %d not supported (F32/F64 only)", dtype);
    if (n_inputs < 1 || n_inputs > NK_FUSED_MAX_IN) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: 1..%d inputs, got %d", NK_FUSED_MAX_IN, n_inputs);
    if (!expr || !*expr) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: empty expression");
    Nvrtc* rt = nvrtc();
    if (!rt->error.empty()) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_compile: run-time compiler unavailable (%s)", rt->error.c_str());

    std::string src;
    src += dtype == NK_F32 ? "typedef float T;\ntypedef float4 V;\n#define VECW 4\n" : "typedef double T;\ntypedef double2 V;\n#define VECW 2\n";
    src += "#define NK_NIN " + std::to_string(n_inputs) + "\n";
    src += "#define NK_EXPR (";
    src += expr;
    src += ")\n";
    src += k_prelude;
    src += k_kernel_src;

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
        return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_compile: the expression does not compile (%s): %s", rt->GetErrorString(rc), log.c_str());
    }
    size_t n = 0;
    rc = rt->GetCUBINSize(prog, &n);
    std::vector<char> image(n);
    if (!rc && n) rc = rt->GetCUBIN(prog, image.data());
    rt->DestroyProgram(&prog);
    if (rc || !n) return nk_fail(ctx, NK_ERR_CUDA, "nk_fused_compile: no device image (%s)", rc ? rt->GetErrorString(rc) : "empty");

    nk_fused* f = new (std::nothrow) nk_fused();
    if (!f) return nk_fail(ctx, NK_ERR_OOM, "nk_fused_compile: out of host memory");
    cudaError_t e = cudaLibraryLoadData(&f->lib, image.data(), nullptr, nullptr, 0, nullptr, nullptr, 0);
    if (e == cudaSuccess) e = cudaLibraryGetKernel(&f->kernel, f->lib, "nk_fused_kernel");
    if (e != cudaSuccess) {
        if (f->lib) cudaLibraryUnload(f->lib);
        delete f;
        return nk_cuda_fail(ctx, e, "cudaLibraryLoadData / cudaLibraryGetKernel (fused kernel)");
    }
    f->dtype = dtype;
    f->n_in = n_inputs;
    f->device = ctx->device;
    *out = f;
    return NK_OK;
}

static bool nk_fused_needs_wide(int64_t units, int64_t rows, int64_t grid) {
    const int64_t lim = int64_t(1) << 32;
    return units + grid >= lim || rows + 2 >= lim;
}

extern "C" int nk_fused_run(nk_ctx* ctx, nk_fused* f, int32_t rank, nk_buf* drn, const int32_t* cfg0, nk_buf* const* srcs, const int32_t* const* cfgs) {
    NK_CHECK_CTX(ctx);
    if (!f || f->magic != 0x4e4b4655) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: not a fused operation");
    if (f->device != ctx->device) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: compiled for device %d, called on device %d", f->device, ctx->device);
    if (!srcs || !cfgs) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: null operand list");
    NkView v0, v[NK_FUSED_MAX_IN];
    int st;
    if ((st = nk_view_parse(ctx, "nk_fused_run(drain)", drn, cfg0, rank, f->dtype, &v0))) return st;
    for (int j = 0; j < f->n_in; j++)
        if ((st = nk_view_parse(ctx, "nk_fused_run(src)", srcs[j], cfgs[j], rank, f->dtype, &v[j]))) return st;
    if (!v0.imap_row_major)
        return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_fused_run: the drain must be indexed row-major (a fresh output tensor is)");
    // per dim: an operand follows the drain index where it has the drain's extent, stays at 0 where its extent is 1
    // (Broadcast.java:76-95); anything else is a shape error
    FusedArgs a;
    memset(&a, 0, sizeof(a));
    FusedPlan& p = a.p;
    int64_t e[NK_MAX_RANK], s0[NK_MAX_RANK], s[NK_FUSED_MAX_IN][NK_MAX_RANK];
    for (int k = 0; k < rank; k++) {
        e[k] = v0.shape[k];
        s0[k] = v0.estride[k];
        for (int j = 0; j < f->n_in; j++) {
            if (v[j].shape[k] == e[k]) s[j][k] = e[k] == 1 ? 0 : v[j].estride[k];
            else if (v[j].shape[k] == 1) s[j][k] = 0;
            else return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_fused_run: operand %d has extent %lld in dim %d, the drain %lld", j, (long long)v[j].shape[k], k, (long long)e[k]);
        }
    }
    // drop size-1 dims, merge neighbours across which every tensor is linear
    int nd = 0;
    for (int k = 0; k < rank; k++) {
        if (e[k] == 1) continue;
        bool merge = nd > 0 && p.s0[nd - 1] == e[k] * s0[k];
        for (int j = 0; j < f->n_in && merge; j++) merge = p.s[j][nd - 1] == e[k] * s[j][k];
        if (merge) {
            p.ext[nd - 1] *= e[k];
            p.s0[nd - 1] = s0[k];
            for (int j = 0; j < f->n_in; j++) p.s[j][nd - 1] = s[j][k];
        } else {
            p.ext[nd] = e[k];
            p.s0[nd] = s0[k];
            for (int j = 0; j < f->n_in; j++) p.s[j][nd] = s[j][k];
            nd++;
        }
    }
    if (nd == 0) { p.ext[0] = 1; nd = 1; }
    p.nd = nd;
    p.n_in = f->n_in;
    p.b0 = v0.base;
    a.out = drn->ptr;
    for (int j = 0; j < f->n_in; j++) { p.b[j] = v[j].base; a.in[j] = srcs[j]->ptr; }
    // a fully linear problem is one long row: cut it into rows of 1024 so that a thread still has several loads in flight
    if (nd == 1 && p.ext[0] >= 8192 && p.ext[0] % 1024 == 0) {
        p.ext[1] = 1024; p.s0[1] = p.s0[0];
        for (int j = 0; j < f->n_in; j++) p.s[j][1] = p.s[j][0];
        p.ext[0] /= 1024; p.s0[0] *= 1024;
        for (int j = 0; j < f->n_in; j++) p.s[j][0] *= 1024;
        nd = 2;
        p.nd = 2;
    }
    p.inner = p.ext[nd - 1];
    // 128-bit accesses along the innermost dim when everything lines up
    const int es = int(nk_dtype_size(f->dtype)), W = 16 / es;
    bool vec = p.s0[nd - 1] == 1 && p.inner % W == 0 && ((reinterpret_cast<uintptr_t>(drn->ptr) + size_t(p.b0) * es) & 15) == 0;
    for (int k = 0; k < nd - 1 && vec; k++) vec = p.s0[k] % W == 0;
    for (int j = 0; j < f->n_in && vec; j++) {
        const int64_t si = p.s[j][nd - 1];
        if (si != 0 && si != 1) vec = false;
        if (si == 1) {
            if ((reinterpret_cast<uintptr_t>(srcs[j]->ptr) + size_t(p.b[j]) * es) & 15) vec = false;
            for (int k = 0; k < nd - 1 && vec; k++) vec = p.s[j][k] % W == 0;
        }
    }
    p.vec = vec ? W : 1;
    const int64_t per_chunk = 256 * int64_t(p.vec);
    p.chunks = (p.inner + per_chunk - 1) / per_chunk;
    int64_t rows = 1;
    for (int k = 0; k < nd - 1; k++) rows *= p.ext[k];
    p.rows = rows;
    p.units = ((rows + 1) / 2) * p.chunks;   // groups of NK_ROWS = 2 rows
    if (p.units == 0) return NK_OK;
    const int64_t cap = int64_t(ctx->prop.multiProcessorCount) * 16;
    // 32-bit unit and row arithmetic in the kernel only while neither the unit counter (it steps by the grid size) nor
    // the row index of a group's second row can pass 2^32
    p.wide = nk_fused_needs_wide(p.units, rows, cap) ? 1 : 0;
    const unsigned grid = unsigned(p.units < cap ? p.units : cap);
    void* params[] = {&a};
    NK_CUDA(ctx, cudaLaunchKernel(reinterpret_cast<const void*>(f->kernel), dim3(grid), dim3(256), params, 0, ctx->stream));
    return nk_after_launch(ctx, "nk_fused_kernel");
}

// Exported for the host-side test of the plan arithmetic.
extern "C" int nk_fused_plan_is_wide(int64_t units, int64_t rows, int64_t grid) { return nk_fused_needs_wide(units, rows, grid) ? 1 : 0; }

extern "C" int nk_fused_free(nk_fused* f) {
    if (!f || f->magic != 0x4e4b4655) return NK_ERR_BAD_ARG;
    cudaSetDevice(f->device);
    if (f->lib) cudaLibraryUnload(f->lib);
    f->magic = 0;
    delete f;
    return NK_OK;
}
