// java.util.Random-compatible input generator (host side). The 48-bit LCG constants and the polar
// Gaussian are those of Neureka's CPURandomization
// (src/main/java/neureka/backend/main/implementations/elementwise/CPURandomization.java:12-15, :265-307),
// which the reference's own test pins to java.util.Random
// (src/test/groovy/ut/backend/core/Randomization_Spec.groovy:39-54). Streams follow java.util.Random:
// setSeed scrambles with the multiplier, nextFloat uses 24 bits, nextDouble 26+27 bits, nextGaussian
// keeps the second value of each polar pair for the next call.
#include <cmath>
#include <cstdint>
#include "../../include/neureka_cuda.h"

namespace {
constexpr uint64_t MULT = 0x5DEECE66DULL, ADD = 0xBULL, MASK = (1ULL << 48) - 1;
struct JRandom {
    uint64_t seed;
    bool have_next = false;
    double next_gaussian = 0;
    explicit JRandom(int64_t s) : seed((uint64_t(s) ^ MULT) & MASK) {}
    int32_t next(int bits) {
        seed = (seed * MULT + ADD) & MASK;
        return int32_t(int64_t(seed) >> (48 - bits));
    }
    float next_float() { return float(next(24)) / float(1 << 24); }
    double next_double() { return double((int64_t(next(26)) << 27) + next(27)) * 0x1.0p-53; }
    double gaussian() {
        if (have_next) { have_next = false; return next_gaussian; }
        double v1, v2, s;
        do {
            v1 = 2 * next_double() - 1;
            v2 = 2 * next_double() - 1;
            s = v1 * v1 + v2 * v2;
        } while (s >= 1 || s == 0);
        double multiplier = std::sqrt(-2 * std::log(s) / s);
        next_gaussian = v2 * multiplier;
        have_next = true;
        return v1 * multiplier;
    }
};
}  // namespace

// state after `steps` LCG steps: s -> A*s + C with (A, C) = (MULT, ADD) composed `steps` times (mod 2^48)
static uint64_t lcg_jump(uint64_t s, uint64_t steps) {
    uint64_t a = MULT, c = ADD, A = 1, C = 0;
    while (steps) {
        if (steps & 1) { A = (A * a) & MASK; C = (C * a + c) & MASK; }
        c = ((a + 1) * c) & MASK;
        a = (a * a) & MASK;
        steps >>= 1;
    }
    return (A * s + C) & MASK;
}

extern "C" int nk_jrand_fill(int32_t dtype, int32_t dist, int64_t seed, double p0, double p1, void* host_out, int64_t n) {
    return nk_jrand_fill_at(dtype, dist, seed, p0, p1, 0, host_out, n);
}

extern "C" int nk_jrand_fill_at(int32_t dtype, int32_t dist, int64_t seed, double p0, double p1, int64_t start,
                                void* host_out, int64_t n) {
    if (host_out == nullptr || n < 0 || start < 0) return NK_ERR_BAD_ARG;
    if (dtype != NK_F32 && dtype != NK_F64) return NK_ERR_UNSUPPORTED;
    if (dist != 0 && dist != 1) return NK_ERR_BAD_ARG;
    if (dist == 1 && start != 0) return NK_ERR_UNSUPPORTED;   // the polar method consumes a data-dependent number of steps
    JRandom r(seed);
    if (start > 0) r.seed = lcg_jump(r.seed, uint64_t(start) * (dtype == NK_F32 ? 1u : 2u));
    if (dtype == NK_F32) {
        float* o = static_cast<float*>(host_out);
        if (dist == 0) { const float lo = float(p0), w = float(p1 - p0); for (int64_t i = 0; i < n; i++) o[i] = lo + w * r.next_float(); }
        else for (int64_t i = 0; i < n; i++) o[i] = float(p0 + p1 * r.gaussian());
    } else {
        double* o = static_cast<double*>(host_out);
        if (dist == 0) for (int64_t i = 0; i < n; i++) o[i] = p0 + (p1 - p0) * r.next_double();
        else for (int64_t i = 0; i < n; i++) o[i] = p0 + p1 * r.gaussian();
    }
    return NK_OK;
}
