// Host-side planning for nk_conv: turns the three views of a convolution / deconvolution call into a
// per-dimension gather description that every conv kernel family consumes.
//
// Forward (d < 0), AbstractCPUConvolution.java:245-316: O[p] = sum_q A[alpha]*B[beta], per dim
//   a == b : alpha = beta = q            (dim summed away)
//   a >  b : alpha = p + q, beta = q
//   a <  b : alpha = q,     beta = p + q
// Deconvolution (d >= 0), AbstractCPUConvolution.java:319-408: D[p] = sum_q [0 <= tau < s1] T1[tau]*T2[q],
//   tau = (s0 > s1) ? p - q : p + q, q over the whole of T2 -- evaluated here as a gather: the range of q
//   for which tau is inside T1 is computed per output element, nothing else is visited.
//
// Both become: for output index p, q runs over a box [lo_k(p), hi_k(p)] per dim and
//   offA = bA + sum_k p_k*pa_k + q_k*qa_k ,  offB = bB + sum_k p_k*pb_k + q_k*qb_k.
#pragma once
#include "nk_internal.h"

enum : int { NK_BOX_CONST = 0, NK_BOX_MINUS = 1, NK_BOX_PLUS = 2 };

struct ConvPlan {
    int rank;
    int64_t total;                 // drain elements
    int64_t odiv[NK_MAX_RANK];     // decode of the drain's flat index (its indicesMap)
    int64_t s0[NK_MAX_RANK];       // drain element strides
    int64_t oext[NK_MAX_RANK];     // drain extents
    int mode[NK_MAX_RANK];         // how the q-range of dim k depends on p_k
    int64_t n1[NK_MAX_RANK];       // CONST: q in [0, n1); MINUS/PLUS: extent of T1 (s1)
    int64_t n2[NK_MAX_RANK];       // MINUS/PLUS: extent of T2 (s2)
    int64_t pa[NK_MAX_RANK], qa[NK_MAX_RANK], pb[NK_MAX_RANK], qb[NK_MAX_RANK];
    int64_t b0, bA, bB;
    int64_t max_terms;             // upper bound of terms per output element
};

// q-range of one dim for output index p (inclusive bounds; empty when hi < lo)
__host__ __device__ inline void nk_box_range(const ConvPlan& c, int k, int64_t p, int64_t* lo, int64_t* hi) {
    if (c.mode[k] == NK_BOX_CONST) { *lo = 0; *hi = c.n1[k] - 1; }
    else if (c.mode[k] == NK_BOX_MINUS) {   // tau = p - q in [0, s1)
        int64_t l = p - c.n1[k] + 1; *lo = l > 0 ? l : 0;
        int64_t h = c.n2[k] - 1; *hi = h < p ? h : p;
    } else {                                 // tau = p + q in [0, s1)
        *lo = 0;
        int64_t h = c.n1[k] - 1 - p, h2 = c.n2[k] - 1; *hi = h < h2 ? h : h2;
    }
}

inline int nk_conv_make_plan(nk_ctx* ctx, const NkView& v0, const NkView& v1, const NkView& v2, int d, ConvPlan* c) {
    const int rank = v0.rank;
    c->rank = rank;
    c->total = v0.size;
    c->b0 = v0.base; c->bA = v1.base; c->bB = v2.base;
    c->max_terms = 1;
    for (int k = 0; k < rank; k++) {
        c->odiv[k] = v0.imap[k];
        c->s0[k] = v0.estride[k];
        c->oext[k] = v0.shape[k];
        const int64_t a = v1.shape[k], b = v2.shape[k], o = v0.shape[k];
        if (d < 0) {
            const int64_t n = a < b ? a : b, big = a < b ? b : a;
            if (o + n - 1 > big)
                return nk_fail(ctx, NK_ERR_BAD_ARG,
                               "nk_conv: dim %d: drain extent %lld too large for operands %lld and %lld (expected |a-b|+1 = %lld)",
                               k, (long long)o, (long long)a, (long long)b, (long long)(big - n + 1));
            c->mode[k] = NK_BOX_CONST;
            c->n1[k] = n; c->n2[k] = n;
            c->qa[k] = v1.estride[k]; c->qb[k] = v2.estride[k];
            c->pa[k] = (a > b) ? v1.estride[k] : 0;
            c->pb[k] = (a < b) ? v2.estride[k] : 0;
            if (a == b && o != 1)
                return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_conv: dim %d: equal operand extents %lld need a drain extent of 1, got %lld",
                               k, (long long)a, (long long)o);
            c->max_terms *= n;
        } else {
            const int64_t s0 = o, s1 = a, s2 = b;
            c->mode[k] = (s0 > s1) ? NK_BOX_MINUS : NK_BOX_PLUS;
            c->n1[k] = s1; c->n2[k] = s2;
            c->pa[k] = v1.estride[k];
            c->qa[k] = (s0 > s1) ? -v1.estride[k] : v1.estride[k];
            c->pb[k] = 0;
            c->qb[k] = v2.estride[k];
            int64_t m = s2 < s1 ? s2 : s1;
            c->max_terms *= m;
        }
    }
    return NK_OK;
}
