// Contraction-shaped convolution calls: classification of the three views into the index groups of a matrix product
// O[m, n] = sum_k A[m, k] * B[k, n], shared by the FMA family (nk_conv_gemm.cu) and the tensor-core family (nk_conv_tc.cu).
//
// Forward (d < 0, AbstractCPUConvolution.java:245-316), per dim with extents (a, b) of the operands and o of the drain:
//   a == b       -> summed away (k group)          a > 1, b == 1 -> only the first operand spans it (m group)
//   a == 1, b > 1 -> only the second spans it (n group)           anything else is a sliding window: not a contraction.
// Deconvolution (d >= 0, AbstractCPUConvolution.java:319-408), D[p] = sum_q [0 <= tau < s1] T1[tau] * T2[q] with
// tau = (s0 > s1) ? p - q : p + q, per dim with extents (s0, s1, s2) of drain, T1, T2:
//   s2 == 1, s0 == s1 -> q = 0, tau = p: drain and T1 share the dim (m group)
//   s1 == 1, s0 == s2 -> tau = 0 forces q = p: drain and T2 share it (n group)
//   s0 == 1, s1 == s2 -> tau = q for every q: summed over T1 and T2 (k group)
// -- the two gradients of a `convDot` / matrix product (Convolution.java:56-89, MatMulAlgorithm.java:37-59) have this form.
#pragma once
#include "nk_internal.h"

struct GemmDims {
    int n;                      // dims in this group
    int64_t ext[NK_MAX_RANK];
    int64_t sa[NK_MAX_RANK];    // stride in the first table of the group
    int64_t sb[NK_MAX_RANK];    // stride in the second table of the group
};

struct GemmPlan {
    GemmDims m, n, k;           // m: (A, drain)   n: (B, drain)   k: (A, B)
    int64_t M, N, K;
    int64_t bA, bB, bO;
};


// True when the call is a contraction; fills the groups, extents and bases (A = first source, B = second source).
inline bool nk_gemm_classify(const NkView& v0, const NkView& v1, const NkView& v2, int d, GemmPlan* out) {
    GemmPlan& p = *out;
    memset(&p, 0, sizeof(p));
    p.M = p.N = p.K = 1;
    for (int k = 0; k < v0.rank; k++) {
        const int64_t a = v1.shape[k], b = v2.shape[k], o = v0.shape[k];
        GemmDims* g = nullptr;
        int64_t ext = 1, sa = 0, sb = 0;
        if (a == 1 && b == 1) {
            if (o != 1) return false;
            continue;
        }
        if (d < 0) {
            if (a == b) { if (o != 1) return false; g = &p.k; ext = a; sa = v1.estride[k]; sb = v2.estride[k]; }
            else if (b == 1) { if (o != a) return false; g = &p.m; ext = a; sa = v1.estride[k]; sb = v0.estride[k]; }
            else if (a == 1) { if (o != b) return false; g = &p.n; ext = b; sa = v2.estride[k]; sb = v0.estride[k]; }
            else return false;
        } else {
            if (b == 1 && o == a) { g = &p.m; ext = a; sa = v1.estride[k]; sb = v0.estride[k]; }
            else if (a == 1 && o == b) { g = &p.n; ext = b; sa = v2.estride[k]; sb = v0.estride[k]; }
            else if (o == 1 && a == b) { g = &p.k; ext = a; sa = v1.estride[k]; sb = v2.estride[k]; }
            else return false;
        }
        g->ext[g->n] = ext; g->sa[g->n] = sa; g->sb[g->n] = sb; g->n++;
        if (g == &p.m) p.M *= ext; else if (g == &p.n) p.N *= ext; else p.K *= ext;
    }
    p.bA = v1.base; p.bB = v2.base; p.bO = v0.base;
    return true;
}

// Fills the six offset tables [offA_m | offO_m | offB_n | offO_n | offA_k | offB_k] (M, M, N, N, K, K entries).
int nk_gemm_build_tables(nk_ctx* ctx, const GemmPlan& p, int64_t* tab);

// Tensor-core (tcgen05, 3xTF32) family for F32 contractions; *handled stays false when it declines the call.
int nk_conv_tc_try(nk_ctx* ctx, nk_buf* drn, nk_buf* s1, nk_buf* s2, const GemmPlan& p, bool* handled);
