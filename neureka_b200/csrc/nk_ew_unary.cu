// Entry points nk_unary (the 23 activations + AssignLeft's copy) and nk_scalar_binary (tensor op scalar).
// Compiled with -fmad=false (see nk_scalarfun.cuh).

#include "nk_ew_kernels.cuh"

using namespace nkew;

namespace {

#define NK_UNARY_CASE(FUN, DER) \
    case (FUN * 2 + (DER ? 1 : 0)): return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, UnaryFix<T, FUN, DER>{});

// the common activations get compile-time functors (forward; tanh / sig / relu also their derivative)
template <class T>
int launch_unary(nk_ctx* ctx, int fun, bool derive, T* out, const T* in, const EwPlan& p) {
    switch (fun * 2 + (derive ? 1 : 0)) {
        NK_UNARY_CASE(NK_FUN_IDY, false) NK_UNARY_CASE(NK_FUN_RELU, false) NK_UNARY_CASE(NK_FUN_TANH, false) NK_UNARY_CASE(NK_FUN_SIG, false)
        NK_UNARY_CASE(NK_FUN_ABS, false) NK_UNARY_CASE(NK_FUN_QUAD, false) NK_UNARY_CASE(NK_FUN_EXP, false) NK_UNARY_CASE(NK_FUN_GELU, false)
        NK_UNARY_CASE(NK_FUN_SILU, false) NK_UNARY_CASE(NK_FUN_SOFTPLUS, false)
        NK_UNARY_CASE(NK_FUN_TANH, true) NK_UNARY_CASE(NK_FUN_SIG, true) NK_UNARY_CASE(NK_FUN_RELU, true)
        default: break;
    }
    return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, UnaryF<T>{fun, derive});
}

template <class T>
int launch_scalar(nk_ctx* ctx, int op, int d, T value, T* out, const T* in, const EwPlan& p) {
    if (d < 0) {
        switch (op) {
            case NK_OP_ADD: return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, ScalarFix<T, NK_OP_ADD>{value});
            case NK_OP_SUB: return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, ScalarFix<T, NK_OP_SUB>{value});
            case NK_OP_MUL: return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, ScalarFix<T, NK_OP_MUL>{value});
            case NK_OP_DIV: return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, ScalarFix<T, NK_OP_DIV>{value});
            default: break;
        }
    }
    return launch_ew<T, 1>(ctx, out, in, (const T*)nullptr, p, ScalarF<T>{op, d, value});
}

}  // namespace

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
    if (dtype == NK_F32) return launch_unary<float>(ctx, fun, d >= 0, data_of<float>(drn), data_of<float>(src), p);
    return launch_unary<double>(ctx, fun, d >= 0, data_of<double>(drn), data_of<double>(src), p);
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
    if (dtype == NK_F32) return launch_scalar<float>(ctx, op, dd, float(value), data_of<float>(drn), data_of<float>(src), p);
    return launch_scalar<double>(ctx, op, dd, value, data_of<double>(drn), data_of<double>(src), p);
}

