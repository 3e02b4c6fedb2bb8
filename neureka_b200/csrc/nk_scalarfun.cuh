// Device-side scalar math of the elementwise family. The translation unit including this header is
// compiled with -fmad=false: Neureka's CPU implementation is Java, which never contracts a*b+c, and the
// F32 definitions of most functions are "evaluate in double, then cast" -- kept verbatim here so that
// results agree with the reference to the last bit wherever the math library does.
//
// Formulas: src/main/java/neureka/backend/main/implementations/fun/Scalar*.java (one class per function),
// FunUtil.java:8-29 (inverse square root), implementations/fun/api/CPUFun.java:7-9 (float default).
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include "../../include/neureka_cuda.h"

namespace nkf {

__device__ __forceinline__ double inv_sqrt(double x) {
    double xhalf = 0.5 * x;
    long long i = __double_as_longlong(x);
    i = 0x5fe6ec85e7de30daLL - (i >> 1);
    x = __longlong_as_double(i);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    x *= (1.5 - xhalf * x * x);
    return x;
}
__device__ __forceinline__ float inv_sqrt(float x) {
    float xhalf = 0.5f * x;
    int i = __float_as_int(x);
    i = 0x5f3759df - (i >> 1);
    x = __int_as_float(i);
    x *= (1.5f - xhalf * x * x);
    x *= (1.5f - xhalf * x * x);
    return x;
}

#define NKF_SELU_ALPHA 1.6732632423543772848170429916717
#define NKF_SELU_SCALE 1.0507009873554804934193349852946

// cbrt with one Newton step on the exactly computed residual x - y^3: the result is the correctly rounded
// cube root in all but a vanishing fraction of cases, i.e. within half an ulp of what any conforming
// Math.cbrt returns.
__device__ __forceinline__ double cbrt_cr(double x) {
    double y = cbrt(x);
    if (x == 0.0 || !isfinite(x)) return y;
    double y2 = y * y, e2 = fma(y, y, -y2);        // y^2 = y2 + e2
    double y3 = y2 * y, e3 = fma(y2, y, -y3);      // y2*y = y3 + e3
    double r = ((x - y3) - e3) - e2 * y;           // x - y^3
    return y + r / (3.0 * y2);
}

__device__ __forceinline__ double sig64(double x) { return 1.0 / (1.0 + exp(-x)); }
__device__ __forceinline__ double tanh64(double x) { return 2 / (1 + exp(-x * 2)) - 1; }
__device__ __forceinline__ float tanh32_literal(float x) { return float(2 / (1 + exp(double(-x * 2))) - 1); }
// exp(t) for |t| <= 700 without the library routine's range checks and special cases: k = round(t / ln 2) by the 1.5 * 2^52
// trick, a two-step Cody-Waite reduction, the Taylor polynomial of degree 12 on |f| <= ln 2 / 2 (truncation below 2^-51
// relative; for tiny t the last step 1 + f * p rounds once, i.e. correctly) and 2^k added into the exponent field (the
// result stays inside the normal exponent range).
__device__ __forceinline__ double nk_exp_reduced(double t) {
    const double magic = 6755399441055744.0;
    const double kd = fma(t, 1.4426950408889634074, magic);
    const int k = __double2loint(kd);
    const double kf = kd - magic;
    double f = fma(kf, -6.93147180369123816490e-01, t);
    f = fma(kf, -1.90821492927058770002e-10, f);
    double p = 2.08767569878680989792e-09;            // 1/12!
    p = fma(p, f, 2.50521083854417187751e-08);        // 1/11!
    p = fma(p, f, 2.75573192239858906526e-07);        // 1/10!
    p = fma(p, f, 2.75573192239858906526e-06);        // 1/9!
    p = fma(p, f, 2.48015873015873015873e-05);        // 1/8!
    p = fma(p, f, 1.98412698412698412698e-04);        // 1/7!
    p = fma(p, f, 1.38888888888888888889e-03);        // 1/6!
    p = fma(p, f, 8.33333333333333333333e-03);        // 1/5!
    p = fma(p, f, 4.16666666666666666667e-02);        // 1/4!
    p = fma(p, f, 1.66666666666666666667e-01);        // 1/3!
    p = fma(p, f, 0.5);
    p = fma(p, f, 1.0);
    p = fma(p, f, 1.0);
    return __hiloint2double(__double2hiint(p) + (k << 20), __double2loint(p));
}
// The reference's F32 tanh, (float)(2 / (1 + Math.exp(-2x)) - 1) evaluated in double (ScalarTanh.java:24-25). The literal
// form above is bound by instruction issue, not by the FP64 pipe: 75 instructions per element, most of them integer and
// branch work inside the library's exp and the division's fix-up path. tanh32_fast performs the same operations in the
// same order -- exp, 1 + E, 2 / d, - 1, round to float -- with the lean exp and a quotient made of a hardware reciprocal seed
// and two Newton steps: 22 double-precision instructions, straight-line. Both intermediate results are within a few units
// in the last place of a double of the exactly rounded ones, far below the float rounding, so the float result is the
// literal form's except where the double value falls within ~2^-48 of a float rounding boundary (one ulp then; all 2^32
// inputs are checked against the CPU oracle). That margin does not exist for |x| < 2^-26, where the result is the
// cancellation residue of 2 / d - 1 and near-ties of the quotient decide it, nor for NaN (the clamp swallows it):
// tanh32_rare names those inputs, and they take the literal form. Kernels that evaluate several elements per thread call
// the two halves separately (all fast values first, fix-ups after), so that the elements are evaluated side by side and
// share every constant; with the branch between elements the constants were rebuilt in registers for each one.
__device__ __forceinline__ float tanh32_fast(float x) {
    // beyond |2x| = 40 the formula gives exactly -1 / +1 in float; the clamp keeps the scaling inside the exponent range
    const float t = fminf(fmaxf(x * -2.0f, -40.0f), 40.0f);
    const double d = 1.0 + nk_exp_reduced(double(t));
    double r;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(d));
    double e = fma(-d, r, 1.0);
    r = fma(r, e, r);
    e = fma(-d, r, 1.0);
    r = fma(r, e, r);
    return float(fma(2.0, r, -1.0));   // 2r is exact, so this is (2 / d) - 1 with the one rounding the subtraction has
}
__device__ __forceinline__ bool tanh32_rare(float x) { return !(fabsf(x) >= 1.490116119384765625e-08f); }
__device__ __forceinline__ float tanh32(float x) {
    float y = tanh32_fast(x);
    if (tanh32_rare(x)) y = tanh32_literal(x);
    return y;
}
// The sigmoid inside the F32 functions sig, silu and gelu: 1 / (1 + Math.exp(-a)) in double (ScalarSigmoid.java,
// ScalarSiLU.java, ScalarGeLU.java), evaluated like tanh32_fast -- lean exp, Newton reciprocal, straight line, no
// cancellation and therefore no literal branch. `a` must lie within +-700 (the lean exp's exponent arithmetic); the callers
// clamp the float they start from, which changes no float result: the sigmoid is 1 to the last bit above 37, and below
// -700 it and its product with any float underflow to zero. The clamp swallows a NaN, and -inf * 0 is a NaN in silu and
// gelu: the callers put those back. All 2^32 inputs of sig, every 16th of silu and gelu were checked against the oracle.
__device__ __forceinline__ double sig_lean(double a) {
    const double d = 1.0 + nk_exp_reduced(-a);
    double r;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(r) : "d"(d));
    double e = fma(-d, r, 1.0);
    r = fma(r, e, r);
    e = fma(-d, r, 1.0);
    return fma(r, e, r);
}
__device__ __forceinline__ float sig32(float x) {
    const float y = float(sig_lean(double(fminf(fmaxf(x, -700.0f), 700.0f))));
    return x != x ? x + x : y;
}
__device__ __forceinline__ float silu32(float x) {
    const float y = float(double(x) * sig_lean(double(fminf(fmaxf(x, -700.0f), 700.0f))));
    return (x != x || x == __int_as_float(0xff800000)) ? x - x : y;
}
__device__ __forceinline__ float gelu32(float x) {
    const float y = float(double(x) * sig_lean(double(fminf(fmaxf(x, -411.0f), 411.0f)) * 1.702));
    return (x != x || x == __int_as_float(0xff800000)) ? x - x : y;
}
__device__ __forceinline__ double softsign64(double x) { return x / (1.0 + fabs(x)); }
__device__ __forceinline__ float softsign32(float x) { return x / (1.0f + fabsf(x)); }
__device__ __forceinline__ double selu64(double x) {
    if (x > 0) return NKF_SELU_SCALE * x;
    else if (x <= 0) return NKF_SELU_SCALE * NKF_SELU_ALPHA * (exp(x) - 1);
    else return double(__int_as_float(0x7fc00000));
}

__device__ __forceinline__ double fun(int f, bool derive, double x) {
    if (!derive) switch (f) {
        case NK_FUN_ABS: return fabs(x);
        case NK_FUN_CBRT: return cbrt_cr(x);
        case NK_FUN_COS: return cos(x);
        case NK_FUN_EXP: return exp(x);
        case NK_FUN_GASU: return softsign64(x * x * x);
        case NK_FUN_GATU: return tanh64(x * x * x);
        case NK_FUN_GAUS: return exp(-(x * x));
        case NK_FUN_FAST_GAUS: return 1 / (1 + x * x);
        case NK_FUN_GELU: return x * sig64(x * 1.702);
        case NK_FUN_IDY: return x;
        case NK_FUN_LOG10: return log10(x);
        case NK_FUN_LN: return log(x);
        case NK_FUN_QUAD: return x * x;
        case NK_FUN_RELU: return x >= 0 ? x : x * .01;
        case NK_FUN_SELU: return selu64(x);
        case NK_FUN_SILU: return x * sig64(x);
        case NK_FUN_SIG: return sig64(x);
        case NK_FUN_SIN: return sin(x);
        case NK_FUN_SOFTPLUS: return log(1.0 + exp(x));
        case NK_FUN_SOFTSIGN: return softsign64(x);
        case NK_FUN_SQRT: return sqrt(x);
        case NK_FUN_TANH: return tanh64(x);
        case NK_FUN_FAST_TANH: return x * inv_sqrt(1.0 + x * x);
    }
    else switch (f) {
        case NK_FUN_ABS: return x < 0 ? -1.0 : 1.0;
        case NK_FUN_CBRT: return 1 / (3 * pow(x, 2.0 / 3.0));
        case NK_FUN_COS: return -sin(x);
        case NK_FUN_EXP: return exp(x);
        case NK_FUN_GASU: { double x2 = x * x, x6 = x2 * x2 * x2; return 3.0 * x2 / (2.0 * x2 * fabs(x) + x6 + 1.0); }
        case NK_FUN_GATU: {
            double x2 = x * x, x3 = x2 * x, temp = 3 * x2, t = tanh64(x3), tanh2 = t * t;
            return -temp * tanh2 + temp;
        }
        case NK_FUN_GAUS: return -2 * x * exp(-(x * x));
        case NK_FUN_FAST_GAUS: { double x2 = x * x; return -2 * x / (x2 * x2 + 2 * x2 + 1); }
        case NK_FUN_GELU: { double s = sig64(x * 1.702), ds = s * (1.0 - s); return s + ds * x * 1.702; }
        case NK_FUN_IDY: return 1;
        case NK_FUN_LOG10: return 1 / (x * log(10.0));
        case NK_FUN_LN: return 1.0 / x;
        case NK_FUN_QUAD: return 2 * x;
        case NK_FUN_RELU: return x >= 0 ? 1 : .01;
        case NK_FUN_SELU:
            if (x > 0) return NKF_SELU_SCALE;
            else if (x <= 0) return NKF_SELU_SCALE * NKF_SELU_ALPHA * exp(x);
            else return __longlong_as_double(0x7ff8000000000000LL);
        case NK_FUN_SILU: { double s = sig64(x); return s + (x * s * (1.0 - s)); }
        case NK_FUN_SIG: { double s = sig64(x); return s * (1 - s); }
        case NK_FUN_SIN: return cos(x);
        case NK_FUN_SOFTPLUS: return 1.0 / (1.0 + exp(-x));
        case NK_FUN_SOFTSIGN: return 1.0 / (2.0 * fabs(x) + x * x + 1.0);
        case NK_FUN_SQRT: return 0.5 * inv_sqrt(x);
        case NK_FUN_TANH: { double t = tanh64(x); return 1 - t * t; }   // Math.pow(t, 2) == t*t
        case NK_FUN_FAST_TANH: { double t1 = x * x, t2 = sqrt(1 + t1); return 1 / (t1 * t2 + t2); }
    }
    return __longlong_as_double(0x7ff8000000000000LL);
}

__device__ __forceinline__ float fun(int f, bool derive, float x) {
    if (!derive) switch (f) {
        case NK_FUN_ABS: return fabsf(x);
        case NK_FUN_CBRT: return float(cbrt_cr(double(x)));
        case NK_FUN_EXP: return float(exp(double(x)));
        case NK_FUN_GASU: return softsign32(x * x * x);
        case NK_FUN_GATU: return tanh32(x * x * x);
        case NK_FUN_FAST_GAUS: return 1 / (1 + x * x);
        case NK_FUN_GELU: return gelu32(x);
        case NK_FUN_IDY: return x;
        case NK_FUN_LOG10: return float(log10(double(x)));
        case NK_FUN_QUAD: return x * x;
        case NK_FUN_RELU: return x >= 0 ? x : x * .01f;
        case NK_FUN_SELU: return float(selu64(double(x)));
        case NK_FUN_SILU: return silu32(x);
        case NK_FUN_SIG: return sig32(x);
        case NK_FUN_SOFTSIGN: return softsign32(x);
        case NK_FUN_SQRT: return float(sqrt(double(x)));
        case NK_FUN_TANH: return tanh32(x);
        case NK_FUN_FAST_TANH: return x * inv_sqrt(1.0f + x * x);
        default: return float(fun(f, false, double(x)));  // cos, gaus, ln, sin, softplus
    }
    else switch (f) {
        case NK_FUN_ABS: return x < 0.0f ? -1.0f : 1.0f;
        case NK_FUN_CBRT: return 1 / (3 * float(pow(double(x), double(2.0f / 3.0f))));
        case NK_FUN_EXP: return float(exp(double(x)));
        case NK_FUN_GASU: { float x2 = x * x, x6 = x2 * x2 * x2; return 3.0f * x2 / (2.0f * x2 * fabsf(x) + x6 + 1.0f); }
        case NK_FUN_GATU: {
            float x2 = x * x, x3 = x2 * x, temp = 3 * x2;
            double t = double(tanh32(x3));
            float tanh2 = float(t * t);
            return -temp * tanh2 + temp;
        }
        case NK_FUN_FAST_GAUS: { float x2 = x * x; return -2 * x / (x2 * x2 + 2 * x2 + 1); }
        case NK_FUN_GELU: { float s = float(sig64(double(x) * 1.702)); float ds = s * (1.0f - s); return s + ds * x * 1.702f; }
        case NK_FUN_IDY: return 1;
        case NK_FUN_LOG10: return 1 / (x * float(log(10.0)));
        case NK_FUN_LN: return 1.0f / x;
        case NK_FUN_QUAD: return 2 * x;
        case NK_FUN_RELU: return x >= 0 ? 1.0f : .01f;
        case NK_FUN_SELU:
            if (x > 0) return float(NKF_SELU_SCALE);
            else if (x <= 0) return float(NKF_SELU_SCALE * NKF_SELU_ALPHA * exp(double(x)));
            else return __int_as_float(0x7fc00000);
        case NK_FUN_SILU: { float s = float(sig64(double(x))); return s + (x * s * (1.0f - s)); }
        case NK_FUN_SIG: { float s = float(sig64(double(x))); return s * (1 - s); }
        case NK_FUN_SOFTSIGN: return 1.0f / (2.0f * fabsf(x) + x * x + 1.0f);
        case NK_FUN_SQRT: return 0.5f * inv_sqrt(x);
        case NK_FUN_TANH: { double t = double(tanh32(x)); return float(1 - t * t); }
        case NK_FUN_FAST_TANH: { float t1 = x * x; float t2 = float(sqrt(double(1 + t1))); return 1 / (t1 * t2 + t2); }
        default: return float(fun(f, true, double(x)));  // cos, gaus, sin, softplus
    }
}

// ---- binary operators ---------------------------------------------------------------------------
// family 0: Broadcast  (CPUBroadcast{Addition,...,Power}.java)
// family 1: BiElementwise (CPUBiElementWise{Addition,...,Power}.java)
// family 2: tensor (op) scalar (CPUScalarBroadcast*.java, CPUScalaBroadcastPower.java)
// Math.pow(b, 2) is written b*b (identical to HotSpot's result for exponent 2).
__device__ __forceinline__ double mod(double a, double b) { return fmod(a, b); }
__device__ __forceinline__ float mod(float a, float b) { return fmodf(a, b); }

template <int FAMILY>
__device__ __forceinline__ double bin(int op, int d, double a, double b) {
    switch (op) {
        case NK_OP_ADD:
            if (FAMILY == 0) return a + b;
            return d >= 0 ? 1.0 : a + b;
        case NK_OP_SUB:
            if (FAMILY == 0) return d == 0 ? a + b : a - b;
            return d == 0 ? 1.0 : (d == 1 ? -1.0 : a - b);
        case NK_OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case NK_OP_DIV:
            if (d == 0) return 1.0 / b;
            if (d == 1) return FAMILY == 1 ? -a / (b * b) : -(a / (b * b));
            return a / b;
        case NK_OP_MOD:
            if (d == 0) return 1.0 / b;
            if (d == 1) return FAMILY == 1 ? -a / (b * b) : -(a / (b * b));
            return mod(a, b);
        case NK_OP_POW:
            if (d == 0) return (FAMILY == 0 ? a : b) * pow(a, b - 1);  // Broadcast multiplies by a (sic)
            if (d == 1) return pow(a, b) * log(a);
            return pow(a, b);
        case NK_OP_IDY: return b;
        case NK_OP_MUL_BOTH: return a * b;
    }
    return __longlong_as_double(0x7ff8000000000000LL);
}

template <int FAMILY>
__device__ __forceinline__ float bin(int op, int d, float a, float b) {
    switch (op) {
        case NK_OP_ADD:
            if (FAMILY == 0) return a + b;
            return d >= 0 ? 1.0f : a + b;
        case NK_OP_SUB:
            if (FAMILY == 0) return d == 0 ? a + b : a - b;
            return d == 0 ? 1.0f : (d == 1 ? -1.0f : a - b);
        case NK_OP_MUL: return d == 0 ? b : (d == 1 ? a : a * b);
        case NK_OP_DIV:
            if (d == 0) return 1.0f / b;
            if (d == 1) return float(-(double(a) / (double(b) * double(b))));
            return a / b;
        case NK_OP_MOD:
            if (d == 0) return 1.0f / b;
            if (d == 1) return float(-(double(a) / (double(b) * double(b))));
            return mod(a, b);
        case NK_OP_POW:
            if (d == 0) return float(double(FAMILY == 0 ? a : b) * pow(double(a), double(b - 1)));
            if (d == 1) return float(pow(double(a), double(b)) * log(double(a)));
            return float(pow(double(a), double(b)));
        case NK_OP_IDY: return b;
        case NK_OP_MUL_BOTH: return a * b;
    }
    return __int_as_float(0x7fc00000);
}

}  // namespace nkf
