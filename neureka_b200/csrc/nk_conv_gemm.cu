// Forward convolutions that are dense contractions: every dim is either summed away (equal extents), or belongs to
// one operand only (the other has extent 1 there). Then O[m, n] = sum_k A[m, k] * B[k, n] with m running over the dims
// only A spans, n over the dims only B spans and k over the summed dims -- `Tensor.convDot` /
// "[M,K,1] x [1,K,N]" of the reference (Tensor_Convolution_Spec.groovy:170-215, CrossDeviceSystemTest.java:95-103).
// The generic gather family computes one output per thread and re-reads both operands through L2 for each of them;
// here a CTA owns a BM x BN output tile, stages BK-deep panels of both operands in shared memory and every thread
// keeps a TM x TN block of sums in registers (8 x 8 for F32: 64 FMAs per four 128-bit shared loads).
//
// Any view works: the three index spaces are flattened on the device into offset tables (one launch), so the panels
// are gathered through offA[m] + offKa[k] / offB[n] + offKb[k] and the tile is scattered through offOm[m] + offOn[n].
// K runs with its last dim fastest, in rising order inside each thread, so the result does not depend on scheduling.
//
// Plain FP32 / FP64 FMAs on purpose: the parity bar is 1e-5 / 1e-12 against a sum in the tensor's own type; FP64
// tensor-core MMA has the same rate as the FP64 FMA pipe on this GPU, and a 3xTF32 tcgen05 pipeline is not built.
#include "nk_gemm_plan.h"

namespace {

// tables: [offA_m | offO_m] (M each), [offB_n | offO_n] (N each), [offA_k | offB_k] (K each)
__global__ void __launch_bounds__(256) nk_gemm_offsets_kernel(int64_t* __restrict__ tab, GemmPlan p) {
    const int64_t total = p.M + p.N + p.K;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += int64_t(gridDim.x) * blockDim.x) {
        const GemmDims* g;
        int64_t idx, *t1, *t2;
        if (i < p.M) { g = &p.m; idx = i; t1 = tab; t2 = tab + p.M; }
        else if (i < p.M + p.N) { g = &p.n; idx = i - p.M; t1 = tab + 2 * p.M; t2 = tab + 2 * p.M + p.N; }
        else { g = &p.k; idx = i - p.M - p.N; t1 = tab + 2 * p.M + 2 * p.N; t2 = tab + 2 * p.M + 2 * p.N + p.K; }
        int64_t rem = idx, a = 0, b = 0;
        for (int d = g->n - 1; d >= 0; d--) {
            const int64_t q = rem % g->ext[d];
            rem /= g->ext[d];
            a += q * g->sa[d];
            b += q * g->sb[d];
        }
        t1[idx] = a;
        t2[idx] = b;
    }
}

}  // namespace

int nk_gemm_build_tables(nk_ctx* ctx, const GemmPlan& p, int64_t* tab) {
    nk_gemm_offsets_kernel<<<nk_grid_for(ctx, p.M + p.N + p.K, 256, 4), 256, 0, ctx->stream>>>(tab, p);
    return nk_after_launch(ctx, "nk_gemm_offsets_kernel");
}

namespace {

template <class T> struct GemmTile;
template <> struct GemmTile<float> { static constexpr int BM = 128, BN = 128, BK = 16, TM = 8, TN = 8; };
template <> struct GemmTile<double> { static constexpr int BM = 128, BN = 64, BK = 8, TM = 8, TN = 4; };

// 256 threads as 16 x 16; thread (ty, tx) owns rows {ty*TM/2 .. +TM/2} of each half of the tile's rows and columns
// {tx*TN/2 .. +TN/2} of each half of its columns, so that the lanes of a quarter warp read consecutive 16-byte words.
// OFF: type the per-thread gather offsets are kept in -- 32 bits when both operands are smaller than 2^31 elements (half the
// registers of the 64-bit form, which spilled inside the main loop).
template <class T, class OFF>
__global__ void __launch_bounds__(256, 2) nk_conv_gemm_kernel(T* __restrict__ out, const T* __restrict__ A, const T* __restrict__ B,
                                                           const int64_t* __restrict__ tab, GemmPlan p) {
    using C = GemmTile<T>;
    constexpr int BM = C::BM, BN = C::BN, BK = C::BK, TM = C::TM, TN = C::TN, HM = TM / 2, HN = TN / 2;
    constexpr int PADM = BM + 4, PADN = BN + 4;
    constexpr int LA = BM * BK / 256, LB = BN * BK / 256;   // elements a thread fetches per panel
    __shared__ __align__(16) T As[2][BK][PADM];
    __shared__ __align__(16) T Bs[2][BK][PADN];

    const int64_t* offA_m = tab;
    const int64_t* offO_m = tab + p.M;
    const int64_t* offB_n = tab + 2 * p.M;
    const int64_t* offO_n = tab + 2 * p.M + p.N;
    const int64_t* offA_k = tab + 2 * p.M + 2 * p.N;
    const int64_t* offB_k = tab + 2 * p.M + 2 * p.N + p.K;

    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t tilesN = (p.N + BN - 1) / BN;
    const int64_t m0 = (blockIdx.x / tilesN) * BM, n0 = (blockIdx.x % tilesN) * BN;

    // panel fetch pattern: A by (m = tid / BK + i * (256 / BK), k = tid % BK) -- k fastest, contiguous for row-major A;
    //                      B by (k = tid / BN + i * (256 / BN), n = tid % BN) -- n fastest, contiguous for row-major B
    const int ak = tid % BK, am = tid / BK;
    const int bn = tid % BN, bk = tid / BN;
    // rows / columns past the edge are clamped to the last valid one (their products land in accumulators that are
    // never stored), so the panel loads need no per-element predicate; only the K tail is guarded
    OFF a_off[LA], b_off;
#pragma unroll
    for (int i = 0; i < LA; i++) {
        int64_t m = m0 + am + i * (256 / BK);
        if (m >= p.M) m = p.M - 1;
        a_off[i] = OFF(p.bA + offA_m[m]);
    }
    {
        int64_t n = n0 + bn;
        if (n >= p.N) n = p.N - 1;
        b_off = OFF(p.bB + offB_n[n]);
    }

    T ra[LA], rb[LB];
    auto fetch = [&](int64_t k0) {
        if (k0 + BK <= p.K) {
            const OFF oka = OFF(offA_k[k0 + ak]);
#pragma unroll
            for (int i = 0; i < LA; i++) ra[i] = A[a_off[i] + oka];
#pragma unroll
            for (int i = 0; i < LB; i++) rb[i] = B[b_off + OFF(offB_k[k0 + bk + i * (256 / BN)])];
        } else {
            const int64_t ka = k0 + ak;
#pragma unroll
            for (int i = 0; i < LA; i++) ra[i] = ka < p.K ? A[a_off[i] + OFF(offA_k[ka])] : T(0);
#pragma unroll
            for (int i = 0; i < LB; i++) {
                const int64_t kb = k0 + bk + i * (256 / BN);
                rb[i] = kb < p.K ? B[b_off + OFF(offB_k[kb])] : T(0);
            }
        }
    };
    auto stash = [&](int buf) {
#pragma unroll
        for (int i = 0; i < LA; i++) As[buf][ak][am + i * (256 / BK)] = ra[i];
#pragma unroll
        for (int i = 0; i < LB; i++) Bs[buf][bk + i * (256 / BN)][bn] = rb[i];
    };

    T acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = T(0);

    fetch(0);
    stash(0);
    __syncthreads();
    int buf = 0;
    for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
        const bool more = k0 + BK < p.K;
        if (more) fetch(k0 + BK);   // global loads of the next panels fly while this one is consumed
#pragma unroll
        for (int k = 0; k < BK; k++) {
            T a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < HM; i++) { a[i] = As[buf][k][ty * HM + i]; a[HM + i] = As[buf][k][BM / 2 + ty * HM + i]; }
#pragma unroll
            for (int j = 0; j < HN; j++) { b[j] = Bs[buf][k][tx * HN + j]; b[HN + j] = Bs[buf][k][BN / 2 + tx * HN + j]; }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fma(a[i], b[j], acc[i][j]);
        }
        if (more) {
            stash(buf ^ 1);   // the other buffer was last read one iteration ago, before the barrier below
            __syncthreads();
            buf ^= 1;
        }
    }

#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int64_t m = m0 + (i < HM ? ty * HM + i : BM / 2 + ty * HM + (i - HM));
        if (m >= p.M) continue;
        const int64_t om = p.bO + offO_m[m];
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int64_t n = n0 + (j < HN ? tx * HN + j : BN / 2 + tx * HN + (j - HN));
            if (n < p.N) out[om + offO_n[n]] = acc[i][j];
        }
    }
}

template <class T>
int launch_gemm(nk_ctx* ctx, T* out, const T* A, const T* B, const GemmPlan& p, bool narrow) {
    using C = GemmTile<T>;
    void* scratch = nullptr;
    const int64_t entries = 2 * (p.M + p.N + p.K);
    int st = nk_scratch(ctx, size_t(entries) * sizeof(int64_t), &scratch);
    if (st) return st;
    int64_t* tab = reinterpret_cast<int64_t*>(scratch);
    st = nk_gemm_build_tables(ctx, p, tab);
    if (st) return st;
    const int64_t tiles = ((p.M + C::BM - 1) / C::BM) * ((p.N + C::BN - 1) / C::BN);
    if (tiles > 0x7fffffffLL) return -1;
    if (narrow) nk_conv_gemm_kernel<T, unsigned><<<unsigned(tiles), 256, 0, ctx->stream>>>(out, A, B, tab, p);
    else nk_conv_gemm_kernel<T, int64_t><<<unsigned(tiles), 256, 0, ctx->stream>>>(out, A, B, tab, p);
    return nk_after_launch(ctx, "nk_conv_gemm_kernel");
}

}  // namespace

// Forward calls and deconvolutions. *handled is set when the call was a contraction and has been launched.
int nk_conv_gemm_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1, nk_buf* s2, const NkView& v2,
                     int d, bool* handled) {
    *handled = false;
    GemmPlan p;
    if (!nk_gemm_classify(v0, v1, v2, d, &p)) return NK_OK;
    // small or skinny problems stay on the gather family (one launch, no tables; a 128-wide tile would be mostly empty)
    const bool forced = ctx->conv_path != NK_CONV_AUTO;   // a forced family skips the "is it worth it" volume test only
    if (p.M < 32 || p.N < 32 || p.K < 16) return NK_OK;
    if (!forced && double(p.M) * double(p.N) * double(p.K) < double(1 << 21)) return NK_OK;
    int st;
    if (dtype == NK_F32 && ctx->conv_path != NK_CONV_GEMM) {   // the tensor-core family first; it declines what it cannot take
        st = nk_conv_tc_try(ctx, drn, s1, s2, p, handled);
        if (st) return st;
        if (*handled) { ctx->last_conv_path = NK_CONV_TC; return NK_OK; }
    }
    if (ctx->conv_path == NK_CONV_TC) return NK_OK;
    const bool narrow = s1->n_elems < (int64_t(1) << 31) && s2->n_elems < (int64_t(1) << 31);   // every gather offset fits 32 bits
    if (dtype == NK_F32) st = launch_gemm<float>(ctx, (float*)drn->ptr, (const float*)s1->ptr, (const float*)s2->ptr, p, narrow);
    else st = launch_gemm<double>(ctx, (double*)drn->ptr, (const double*)s1->ptr, (const double*)s2->ptr, p, narrow);
    if (st == -1) return NK_OK;
    if (st) return st;
    ctx->last_conv_path = NK_CONV_GEMM;
    *handled = true;
    return NK_OK;
}
