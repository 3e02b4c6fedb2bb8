// Deconvolution (d >= 0) whose result is the SMALL, kernel-like tensor -- the gradient of a convolution w.r.t. its
// kernel: D[p] = sum_q T1[p + q] * T2[q], q over the whole (large) T2, p over a window of KH x KW taps (times a few
// outer coordinates). Few outputs, each a reduction over millions of products.
//
// One CTA walks a list of work units; a unit is one TH x TW tile of T2 (the error) for one outer reduction index,
// together with the (TH+KH-1) x (TW+KW-1) tile of T1 (the image) at the same position. Both tiles arrive by TMA
// (zero fill outside the tensors: a missing term contributes 0, exactly like the reference's range check) into two
// shared-memory rings fed by a producer warp (full/empty mbarriers, every wait bounded; the eight compute warps never
// meet a CTA-wide barrier inside the loop). A thread owns RH x CW positions of the error tile, which it copies into
// registers at the start of a unit -- so the error ring's slot is free again at once and needs fewer stages than the
// image ring -- and keeps all KH x KW partial sums in registers; every image row segment it loads feeds up to KH tap
// rows. Small F32 windows run 8 rows per thread (image ring of 2, error ring of 1: two CTAs per SM), the others 4 rows
// (rings of 3 and 3, one barrier pair per slot for both tiles). After its last unit the CTA reduces
// the partial sums (warp shuffles, then the eight warp results in order) and writes one partial window to scratch;
// a second kernel adds the CTAs' windows in CTA order, so the result does not depend on scheduling.
#pragma once
#include "nk_conv_tiled.cuh"

struct WgradPlan {
    int n_outer;
    int64_t oext[NK_MAX_RANK], os[NK_MAX_RANK];   // outer output extents and drain strides
    int64_t qext[NK_MAX_RANK];                    // outer reduction extents (T2's extents)
    int64_t NP;                                   // outer outputs
    int64_t NQ;                                   // outer reduction indices
    int EH, EW;                                   // error tile grid is laid over EH x EW
    int tilesX, tilesY;
    int64_t units;                                // NQ * tilesY * tilesX work units per outer output
    int chunks;                                   // CTAs per outer output
    int has_y;
    int nd;                                       // tensor-map dims (same for both maps)
    int64_t sDy, sDx, bD;                         // drain strides of the window dims and base
    int* status;
};

template <class T, int KH, int KW>
struct WgradCfg {
    static constexpr int CW = 16 / int(sizeof(T));
    static constexpr int RH = (sizeof(T) == 4 && KH * KW <= 25) ? 8 : 4;
    static constexpr int TW = 32 * CW;
    static constexpr int TH = 8 * RH;
    static constexpr int HALO_W = ((KW - 1 + CW - 1) / CW) * CW;
    static constexpr int SW = TW + HALO_W;
    static constexpr int SH = TH + KH - 1;
    static constexpr int NS = CW + HALO_W;
    static constexpr int A_BYTES = ((SH * SW * int(sizeof(T)) + 127) / 128) * 128;
    static constexpr int E_BYTES = ((TH * TW * int(sizeof(T)) + 127) / 128) * 128;
    static constexpr int NA = RH == 8 ? 2 : 3;   // stages of the image ring
    static constexpr int NE = RH == 8 ? 1 : 3;   // stages of the error ring
    static size_t smem_bytes() { return size_t(NA) * A_BYTES + size_t(NE) * E_BYTES + 128 + size_t(8) * KH * KW * sizeof(T); }
};

// 288 threads: warps 0..7 multiply, warp 8 feeds the rings. A full barrier completes when its tile has landed (one
// arrival + the tile's bytes), an empty barrier when all eight compute warps are done with the slot. Every wait is bounded.
template <class T, int KH, int KW>
__global__ void __launch_bounds__(288) nk_conv_wgrad_kernel(T* __restrict__ partial, const WgradPlan p,
                                                            const __grid_constant__ CUtensorMap mapA,
                                                            const __grid_constant__ CUtensorMap mapE) {
    using C = WgradCfg<T, KH, KW>;
    constexpr int CW = C::CW, RH = C::RH, TW = C::TW, TH = C::TH, SW = C::SW, SH = C::SH, NS = C::NS, NA = C::NA, NE = C::NE;
    constexpr bool COUPLED = NA == NE;
    extern __shared__ __align__(128) unsigned char nk_smem[];
    unsigned char* a_base = nk_smem;
    unsigned char* e_base = nk_smem + size_t(NA) * C::A_BYTES;
    uint64_t* full_a = reinterpret_cast<uint64_t*>(nk_smem + size_t(NA) * C::A_BYTES + size_t(NE) * C::E_BYTES);
    uint64_t* empty_a = full_a + NA;
    uint64_t* full_e = empty_a + NA;
    uint64_t* empty_e = full_e + NE;
    volatile int* abort_word = reinterpret_cast<volatile int*>(empty_e + NE);   // 2 (NA + NE) <= 10 barriers: inside the 128 bytes
    T* red = reinterpret_cast<T*>(nk_smem + size_t(NA) * C::A_BYTES + size_t(NE) * C::E_BYTES + 128);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t pflat = blockIdx.x / p.chunks;
    const int chunk = int(blockIdx.x % p.chunks);
    const int64_t per = (p.units + p.chunks - 1) / p.chunks;
    const int64_t u_begin = per * chunk;
    const int64_t u_end = (u_begin + per < p.units) ? u_begin + per : p.units;
    const int64_t n_it = u_end > u_begin ? u_end - u_begin : 0;

    if (tid == 256) {
        for (int s = 0; s < NA; s++) { nk_mbar_init(&full_a[s], 1); nk_mbar_init(&empty_a[s], 8); }
        for (int s = 0; s < NE; s++) { nk_mbar_init(&full_e[s], 1); nk_mbar_init(&empty_e[s], 8); }
        *abort_word = 0;
        nk_fence_barrier_init();
    }
    __syncthreads();

    auto wait_or_abort = [&](uint64_t* bar, unsigned parity) -> bool {
        const int r = nk_mbar_wait_bounded(bar, parity, NK_WAIT_LIMIT_NS, abort_word);
        if (r < 0) {
            *abort_word = 1;
            if (p.status) atomicExch(p.status, 1);
        }
        return r > 0;
    };

    T acc[KH][KW];
#pragma unroll
    for (int a = 0; a < KH; a++)
#pragma unroll
        for (int b = 0; b < KW; b++) acc[a][b] = T(0);

    if (warp == 8) {
        if (lane == 0 && n_it > 0) {
            // The unit index is a mixed-radix number (tile x | tile y | outer reduction indices, last dim fastest): taken
            // apart once, then counted up -- the producer shares an issue port with compute warps, so no division per unit.
            int pidx[NK_TILED_MAX_OUTER], q[NK_TILED_MAX_OUTER];
            {
                int64_t rem = pflat;
                for (int k = p.n_outer - 1; k >= 0; k--) { pidx[k] = int(rem % p.oext[k]); rem /= p.oext[k]; }
                rem = u_begin;
                const int tx0 = int(rem % p.tilesX); rem /= p.tilesX;
                const int ty0 = int(rem % p.tilesY); rem /= p.tilesY;
                for (int k = p.n_outer - 1; k >= 0; k--) { q[k] = int(rem % p.qext[k]); rem /= p.qext[k]; }
                int tx = tx0, ty = ty0;
                const unsigned bytes_a = unsigned((p.has_y ? SH : 1) * SW * sizeof(T));
                const unsigned bytes_e = unsigned((p.has_y ? TH : 1) * TW * sizeof(T));
                nk_fence_proxy_async();
                bool ok = true;
                int64_t issued_a = 0, issued_e = 0;
                for (int64_t it = 0; it < n_it && ok; it++) {
                    const int sa = int(it % NA), se = int(it % NE);
                    int ca[5], ce[5];
                    ca[0] = ce[0] = tx * TW;
                    int n = 1;
                    if (p.has_y) { ca[n] = ce[n] = ty * TH; n++; }
                    for (int k = p.n_outer - 1; k >= 0; k--) { ce[n] = q[k]; ca[n] = pidx[k] + q[k]; n++; }
                    if constexpr (COUPLED) {   // rings of equal depth: one barrier pair per slot serves both tiles
                        if (it >= NA) ok = wait_or_abort(&empty_a[sa], unsigned(it / NA - 1) & 1u);
                        if (!ok) break;
                        nk_mbar_expect_tx(&full_a[sa], bytes_a + bytes_e);
                        nk_tma_load(a_base + size_t(sa) * C::A_BYTES, &mapA, &full_a[sa], p.nd, ca);
                        nk_tma_load(e_base + size_t(se) * C::E_BYTES, &mapE, &full_a[sa], p.nd, ce);
                        issued_a++;
                    } else {
                        // the error slot comes free first (its readers copy it into registers when they start the unit before)
                        if (it >= NE) ok = wait_or_abort(&empty_e[se], unsigned(it / NE - 1) & 1u);
                        if (!ok) break;
                        nk_mbar_expect_tx(&full_e[se], bytes_e);
                        nk_tma_load(e_base + size_t(se) * C::E_BYTES, &mapE, &full_e[se], p.nd, ce);
                        issued_e++;
                        if (it >= NA) ok = wait_or_abort(&empty_a[sa], unsigned(it / NA - 1) & 1u);
                        if (!ok) break;
                        nk_mbar_expect_tx(&full_a[sa], bytes_a);
                        nk_tma_load(a_base + size_t(sa) * C::A_BYTES, &mapA, &full_a[sa], p.nd, ca);
                        issued_a++;
                    }
                    if (++tx == p.tilesX) {
                        tx = 0;
                        if (++ty == p.tilesY) {
                            ty = 0;
                            for (int k = p.n_outer - 1; k >= 0; k--) {
                                if (++q[k] < int(p.qext[k])) break;
                                q[k] = 0;
                            }
                        }
                    }
                }
                if (!ok || *abort_word) {
                    // requested copies may still be landing in this CTA's shared memory: wait for the last ones (bounded)
                    for (int64_t j = (issued_a > NA ? issued_a - NA : 0); j < issued_a; j++)
                        nk_mbar_wait_bounded(&full_a[j % NA], unsigned(j / NA) & 1u, NK_WAIT_LIMIT_NS, nullptr);
                    for (int64_t j = (issued_e > NE ? issued_e - NE : 0); j < issued_e; j++)
                        nk_mbar_wait_bounded(&full_e[j % NE], unsigned(j / NE) & 1u, NK_WAIT_LIMIT_NS, nullptr);
                }
            }
        }
    } else {
        // when the maps have no row dim only row 0 of each tile is real: rows beyond it must not contribute
        const int rows = p.has_y ? RH : (warp == 0 ? 1 : 0);
        for (int64_t it = 0; it < n_it; it++) {
            const int sa = int(it % NA), se = int(it % NE);
            // this thread's error values into registers, and the error slot goes back to the producer
            if (!wait_or_abort(COUPLED ? &full_a[sa] : &full_e[se], unsigned(it / NE) & 1u)) break;
            T ev[RH][CW];
            auto load_ev = [&]() {
                const T* et = reinterpret_cast<const T*>(e_base + size_t(se) * C::E_BYTES) + (warp * RH) * TW + lane * CW;
#pragma unroll
                for (int i = 0; i < RH; i++) {
                    if (i < rows) {
                        if (sizeof(T) == 4) *reinterpret_cast<float4*>(ev[i]) = *reinterpret_cast<const float4*>(et + i * TW);
                        else *reinterpret_cast<double2*>(ev[i]) = *reinterpret_cast<const double2*>(et + i * TW);
                    } else {
#pragma unroll
                        for (int x = 0; x < CW; x++) ev[i][x] = T(0);
                    }
                }
            };
            if constexpr (!COUPLED) {
                load_ev();
                __syncwarp();
                if (lane == 0) nk_mbar_arrive(&empty_e[se]);
                if (!wait_or_abort(&full_a[sa], unsigned(it / NA) & 1u)) break;
            }
            if (rows > 0) {
                if constexpr (COUPLED) load_ev();   // (inside the branch: the row loads below are scheduled together with these)
                const T* at = reinterpret_cast<const T*>(a_base + size_t(sa) * C::A_BYTES) + (warp * RH) * SW + lane * CW;
#pragma unroll
                for (int j = 0; j < RH + KH - 1; j++) {
                    if (!p.has_y && j > 0) break;
                    T seg[NS];
#pragma unroll
                    for (int v = 0; v < NS / CW; v++) {
                        if (sizeof(T) == 4) *reinterpret_cast<float4*>(&seg[v * CW]) = *reinterpret_cast<const float4*>(at + j * SW + v * CW);
                        else *reinterpret_cast<double2*>(&seg[v * CW]) = *reinterpret_cast<const double2*>(at + j * SW + v * CW);
                    }
#pragma unroll
                    for (int ky = 0; ky < KH; ky++) {
                        const int i = j - ky;   // error row that meets image row j at tap row ky
                        if (i >= 0 && i < RH) {
#pragma unroll
                            for (int kx = 0; kx < KW; kx++)
#pragma unroll
                                for (int x = 0; x < CW; x++) acc[ky][kx] = fma(seg[kx + x], ev[i][x], acc[ky][kx]);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) nk_mbar_arrive(&empty_a[sa]);
        }
    }
    __syncthreads();
    if (*abort_word) return;

    // ---- CTA reduction: lanes by shuffle (fixed tree), then the 8 warps in order ----------------------------------
    if (warp < 8) {
#pragma unroll
        for (int a = 0; a < KH; a++)
#pragma unroll
            for (int b = 0; b < KW; b++) {
                T v = acc[a][b];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
                if (lane == 0) red[warp * KH * KW + a * KW + b] = v;
            }
    }
    __syncthreads();
    if (tid < KH * KW) {
        T total = 0;
        for (int w = 0; w < 8; w++) total += red[w * KH * KW + tid];
        partial[(pflat * p.chunks + chunk) * int64_t(KH * KW) + tid] = total;
    }
}

// One warp per kernel tap: lane l adds chunks l, l+32, ... in rising order, then the 32 lane sums are folded by a
// fixed shuffle tree, so the result does not depend on scheduling (run-to-run deterministic).
template <class T>
__global__ void __launch_bounds__(128) nk_conv_wgrad_finish_kernel(T* __restrict__ out, const T* __restrict__ partial, WgradPlan p, int KH, int KW) {
    const int64_t i = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int win = KH * KW;
    if (i >= p.NP * win) return;   // warp-uniform
    const int64_t pflat = i / win;
    const int t = int(i % win);
    T total = 0;
    for (int c = lane; c < p.chunks; c += 32) total += partial[(pflat * p.chunks + c) * int64_t(win) + t];
#pragma unroll
    for (int s = 16; s > 0; s >>= 1) total += __shfl_down_sync(0xffffffffu, total, s);
    if (lane) return;
    int64_t o = p.bD + (t / KW) * p.sDy + (t % KW) * p.sDx;
    int64_t rem = pflat;
    for (int k = p.n_outer - 1; k >= 0; k--) { o += (rem % p.oext[k]) * p.os[k]; rem /= p.oext[k]; }
    out[o] = total;
}

template <class T, int KH, int KW>
int nk_launch_wgrad(nk_ctx* ctx, T* out, WgradPlan& p, const TmaImage& imgA, const TmaImage& imgE) {
    using C = WgradCfg<T, KH, KW>;
    const size_t smem = C::smem_bytes();
    if (smem > size_t(ctx->prop.sharedMemPerBlockOptin) || C::SW > 256 || C::SH > 256) return -1;
    p.tilesX = (p.EW + C::TW - 1) / C::TW;
    p.tilesY = p.has_y ? (p.EH + C::TH - 1) / C::TH : 1;
    p.units = p.NQ * int64_t(p.tilesY) * p.tilesX;
    cudaError_t e = cudaFuncSetAttribute(nk_conv_wgrad_kernel<T, KH, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaFuncSetAttribute(nk_conv_wgrad_kernel)");
    // as many CTAs as are resident at once (KH*KW accumulators per thread decide that), so that the grid is one wave
    int per_sm = 1;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, nk_conv_wgrad_kernel<T, KH, KW>, 288, smem);
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor(nk_conv_wgrad_kernel)");
    if (per_sm < 1) per_sm = 1;
    int64_t chunks = int64_t(ctx->prop.multiProcessorCount) * per_sm / p.NP;
    if (chunks > p.units) chunks = p.units;
    if (chunks > 4096) chunks = 4096;
    if (chunks < 1) chunks = 1;
    p.chunks = int(chunks);
    if (p.NP * chunks > 0x7fffffffLL) return -1;
    const int dt = sizeof(T) == 4 ? NK_F32 : NK_F64;
    CUtensorMap mapA, mapE;
    int st = nk_tma_encode(ctx, dt, imgA, C::SW, C::SH, p.has_y != 0, &mapA);
    if (st) return st;
    st = nk_tma_encode(ctx, dt, imgE, C::TW, C::TH, p.has_y != 0, &mapE);
    if (st) return st;
    void* scratch = nullptr;
    st = nk_scratch(ctx, size_t(p.NP) * size_t(chunks) * KH * KW * sizeof(T), &scratch);
    if (st) return st;
    p.status = ctx->tma_status_dev;
    nk_conv_wgrad_kernel<T, KH, KW><<<unsigned(p.NP * chunks), 288, smem, ctx->stream>>>(reinterpret_cast<T*>(scratch), p, mapA, mapE);
    st = nk_after_launch(ctx, "nk_conv_wgrad_kernel");
    if (st) return st;
    const int64_t n = p.NP * KH * KW;
    nk_conv_wgrad_finish_kernel<T><<<unsigned((n + 3) / 4), 128, 0, ctx->stream>>>(out, reinterpret_cast<const T*>(scratch), p, KH, KW);
    return nk_after_launch(ctx, "nk_conv_wgrad_finish_kernel");
}
