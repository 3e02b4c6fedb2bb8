// Tiled direct-stencil convolution (forward, d < 0) for dense image-like calls.
//
// Shape of the work: one operand (the "image") is larger than the other (the "kernel") in the last one or two
// dims, which therefore slide (a window of KH x KW taps); every other dim is handled by the generic per-dim
// rules of the forward convolution -- it may be batch-like (kernel extent 1), summed away (equal extents,
// "channels"), an outer window (both > 1) or follow the kernel (image extent smaller) -- and is either part of
// the CTA's output coordinate or of its reduction loop.
//
// One CTA produces a TH x TW output tile for one outer output coordinate and walks the reduction loop
// ("channels") with a multi-stage shared-memory pipeline: the (TH+KH-1) x (TW+KW-1) image tile of channel c+2
// is in flight (cp.async, 16-byte chunks, zero-filled past the image edge) while channel c is consumed. A
// thread owns RH x CW outputs (CW = one 128-bit vector) and slides over the tile rows so that every
// shared-memory row segment it loads feeds up to KH output rows; the KH x KW weights of the current channel
// sit in registers. Each input byte is fetched from HBM once per tile (+ halo); with few tiles and many
// channels the channel range is split across CTAs and a second pass adds the partial planes in a fixed order.
#pragma once
#include "nk_conv_plan.h"

#define NK_TILED_MAX_OUTER 6

struct TiledPlan {
    int n_outer;
    int64_t oext[NK_MAX_RANK], os[NK_MAX_RANK];       // outer output extents / strides
    int64_t pI[NK_MAX_RANK], pK[NK_MAX_RANK];         // image / kernel stride applied to the outer output index
    int64_t qext[NK_MAX_RANK], qI[NK_MAX_RANK], qK[NK_MAX_RANK];  // reduction loop extents / strides
    int64_t NP;    // product of oext
    int NQ;        // product of qext  (channels walked by one CTA group)
    int IH, IW, OH, OW;
    int64_t sIy, sKy, sKx, sOy;
    int64_t bI, bK, bO;
    int tilesX, tilesY, splits;
    int vec;       // 16-byte global->shared copies are legal for every chunk
    int vec_out;   // 16-byte stores to the drain are legal
};

__device__ __forceinline__ void nk_cp_async_16(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_8(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_4(void* smem, const void* gmem, int src_bytes) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(s), "l"(gmem), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void nk_cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void nk_cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

template <class T, int KH, int KW>
struct TiledCfg {
    static constexpr int CW = 16 / int(sizeof(T));            // outputs per thread along x = one 128-bit vector
    static constexpr int RH = 4;                              // output rows per thread
    static constexpr int WARPS = 8;
    static constexpr int TW = 32 * CW;
    static constexpr int TH = WARPS * RH;
    static constexpr int HALO_W = ((KW - 1 + CW - 1) / CW) * CW;
    static constexpr int SW = TW + HALO_W;                    // shared row length, a multiple of CW
    static constexpr int SH = TH + KH - 1;
    static constexpr int STAGES = 3;
    static constexpr int NS = CW + HALO_W;                    // row-segment values a thread loads
    static constexpr int WPAD = ((KH * KW + CW - 1) / CW) * CW;
    static constexpr bool WREG = KH * KW * int(sizeof(T)) <= 200;   // weights of one channel live in registers
    static size_t smem_bytes(int NQ) {
        return size_t(STAGES) * SH * SW * sizeof(T) + size_t(NQ) * WPAD * sizeof(T) + size_t(NQ) * 2 * sizeof(int64_t);
    }
};

template <class T, int KH, int KW>
__global__ void __launch_bounds__(256) nk_conv_tiled_kernel(T* __restrict__ out, T* __restrict__ partial,
                                                            const T* __restrict__ I, const T* __restrict__ K, TiledPlan p) {
    using C = TiledCfg<T, KH, KW>;
    constexpr int CW = C::CW, RH = C::RH, TW = C::TW, TH = C::TH, SW = C::SW, SH = C::SH, STAGES = C::STAGES, NS = C::NS, WPAD = C::WPAD;
    extern __shared__ __align__(16) unsigned char nk_smem[];
    T* tiles = reinterpret_cast<T*>(nk_smem);
    T* wsm = tiles + STAGES * SH * SW;
    int64_t* ioff = reinterpret_cast<int64_t*>(wsm + size_t(p.NQ) * WPAD);   // image offset of channel c

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which tile / outer coordinate / channel range ------------------------------------------------
    int64_t bid = blockIdx.x;
    const int tx = int(bid % p.tilesX); bid /= p.tilesX;
    const int ty = int(bid % p.tilesY); bid /= p.tilesY;
    const int split = int(bid % p.splits); bid /= p.splits;
    const int64_t pflat = bid;
    int64_t baseI = p.bI, baseK = p.bK, baseO = p.bO;
    {
        int64_t rem = pflat;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            int64_t idx = rem % p.oext[k];
            rem /= p.oext[k];
            baseI += idx * p.pI[k]; baseK += idx * p.pK[k]; baseO += idx * p.os[k];
        }
    }
    const int x0 = tx * TW, y0 = ty * TH;
    const int cper = (p.NQ + p.splits - 1) / p.splits;
    const int c_begin = split * cper;
    const int c_end = (c_begin + cper < p.NQ) ? c_begin + cper : p.NQ;

    // ---- stage the channel offsets and this CTA's weights ---------------------------------------------
    for (int c = c_begin + tid; c < c_end; c += blockDim.x) {
        int rem = c;
        int64_t oi = 0, ok = 0;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            int q = rem % int(p.qext[k]);
            rem /= int(p.qext[k]);
            oi += q * p.qI[k]; ok += q * p.qK[k];
        }
        ioff[c] = oi;
        ioff[p.NQ + c] = ok;
    }
    __syncthreads();
    for (int e = tid; e < (c_end - c_begin) * WPAD; e += blockDim.x) {
        const int c = c_begin + e / WPAD, t = e % WPAD;
        T v = 0;
        if (t < KH * KW) v = K[baseK + ioff[p.NQ + c] + (t / KW) * p.sKy + (t % KW) * p.sKx];
        wsm[size_t(c) * WPAD + t] = v;
    }

    // ---- image tile loader ----------------------------------------------------------------------------
    auto load_stage = [&](int stage, int c) {
        T* dst = tiles + stage * SH * SW;
        const T* src = I + baseI + ioff[c];
        constexpr int CPR = SW / CW;   // chunks per row
        for (int id = tid; id < SH * CPR; id += 256) {
            const int row = id / CPR, col = (id - row * CPR) * CW;
            const int gy = y0 + row, gx = x0 + col;
            int valid = (gy < p.IH) ? (p.IW - gx) : 0;
            valid = valid < 0 ? 0 : (valid > CW ? CW : valid);
            const T* g = src + (valid > 0 ? (int64_t(gy) * p.sIy + gx) : 0);
            T* s = dst + row * SW + col;
            if (p.vec) {
                nk_cp_async_16(s, g, valid * int(sizeof(T)));
            } else {
#pragma unroll
                for (int e = 0; e < CW; e++) {
                    const int ok = e < valid ? int(sizeof(T)) : 0;
                    if (sizeof(T) == 4) nk_cp_async_4(s + e, g + (ok ? e : 0), ok);
                    else nk_cp_async_8(s + e, g + (ok ? e : 0), ok);
                }
            }
        }
    };

    T acc[RH][CW];
#pragma unroll
    for (int i = 0; i < RH; i++)
#pragma unroll
        for (int x = 0; x < CW; x++) acc[i][x] = T(0);

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (c_begin + s < c_end) load_stage(s, c_begin + s);
        nk_cp_async_commit();
    }

    for (int c = c_begin; c < c_end; c++) {
        nk_cp_async_wait<STAGES - 2>();
        __syncthreads();   // tile c has landed for everyone; everyone is done reading the stage refilled below
        {
            const int nxt = c + STAGES - 1;
            if (nxt < c_end) load_stage((nxt - c_begin) % STAGES, nxt);
            nk_cp_async_commit();
        }
        const T* tile = tiles + ((c - c_begin) % STAGES) * SH * SW + (warp * RH) * SW + lane * CW;
        const T* wc = wsm + size_t(c) * WPAD;
        T w[C::WREG ? KH * KW : 1];
        if (C::WREG) {
#pragma unroll
            for (int t = 0; t < KH * KW; t++) w[t] = wc[t];
        }
#pragma unroll
        for (int j = 0; j < RH + KH - 1; j++) {
            T seg[NS];
#pragma unroll
            for (int v = 0; v < NS / CW; v++) {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(&seg[v * CW]) = *reinterpret_cast<const float4*>(tile + j * SW + v * CW);
                else *reinterpret_cast<double2*>(&seg[v * CW]) = *reinterpret_cast<const double2*>(tile + j * SW + v * CW);
            }
#pragma unroll
            for (int i = 0; i < RH; i++) {
                const int ky = j - i;
                if (ky >= 0 && ky < KH) {
#pragma unroll
                    for (int kx = 0; kx < KW; kx++) {
                        const T wv = C::WREG ? w[ky * KW + kx] : wc[ky * KW + kx];
#pragma unroll
                        for (int x = 0; x < CW; x++) acc[i][x] = fma(seg[kx + x], wv, acc[i][x]);
                    }
                }
            }
        }
    }
    nk_cp_async_wait<0>();

    // ---- epilogue ---------------------------------------------------------------------------------------
    const int ox = x0 + lane * CW;
#pragma unroll
    for (int i = 0; i < RH; i++) {
        const int oy = y0 + warp * RH + i;
        if (oy >= p.OH || ox >= p.OW) continue;
        T* dst;
        bool vec_ok;
        if (p.splits == 1) {
            dst = out + baseO + int64_t(oy) * p.sOy + ox;
            vec_ok = p.vec_out != 0;
        } else {
            dst = partial + ((int64_t(split) * p.NP + pflat) * p.OH + oy) * int64_t(p.OW) + ox;
            vec_ok = (p.OW % CW) == 0;
        }
        if (vec_ok && ox + CW <= p.OW) {
            if (sizeof(T) == 4) *reinterpret_cast<float4*>(dst) = *reinterpret_cast<float4*>(&acc[i][0]);
            else *reinterpret_cast<double2*>(dst) = *reinterpret_cast<double2*>(&acc[i][0]);
        } else {
#pragma unroll
            for (int x = 0; x < CW; x++)
                if (ox + x < p.OW) dst[x] = acc[i][x];
        }
    }
}

// Adds the partial planes of a channel-split launch in split order (deterministic) and scatters into the drain.
template <class T>
__global__ void __launch_bounds__(256) nk_conv_tiled_finish_kernel(T* __restrict__ out, const T* __restrict__ partial, TiledPlan p) {
    const int64_t plane = p.NP * int64_t(p.OH) * p.OW;
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < plane; i += stride) {
        T total = 0;
        for (int s = 0; s < p.splits; s++) total += partial[int64_t(s) * plane + i];
        const int x = int(i % p.OW);
        int64_t rem = i / p.OW;
        const int y = int(rem % p.OH);
        rem /= p.OH;
        int64_t o = p.bO + int64_t(y) * p.sOy + x;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            o += (rem % p.oext[k]) * p.os[k];
            rem /= p.oext[k];
        }
        out[o] = total;
    }
}

template <class T, int KH, int KW>
int nk_launch_tiled(nk_ctx* ctx, T* out, const T* I, const T* K, TiledPlan& p) {
    using C = TiledCfg<T, KH, KW>;
    const size_t smem = C::smem_bytes(p.NQ);
    if (smem > size_t(ctx->prop.sharedMemPerBlockOptin)) return -1;   // caller falls back to the generic family
    p.tilesX = (p.OW + C::TW - 1) / C::TW;
    p.tilesY = (p.OH + C::TH - 1) / C::TH;
    const int64_t tiles = int64_t(p.tilesX) * p.tilesY * p.NP;
    // channel split: only when the tiles alone cannot fill the machine and each part keeps >= 4 channels
    const int64_t want_ctas = int64_t(ctx->prop.multiProcessorCount) * 2;
    int splits = 1;
    if (tiles < want_ctas && p.NQ >= 8) {
        splits = int((want_ctas + tiles - 1) / tiles);
        if (splits > p.NQ / 4) splits = p.NQ / 4;
        if (splits > 32) splits = 32;
        if (splits < 1) splits = 1;
    }
    p.splits = splits;
    T* partial = nullptr;
    if (splits > 1) {
        void* scratch = nullptr;
        const size_t need = size_t(splits) * size_t(p.NP) * p.OH * p.OW * sizeof(T);
        int st = nk_scratch(ctx, need, &scratch);
        if (st) return st;
        partial = reinterpret_cast<T*>(scratch);
    }
    const int64_t grid = tiles * splits;
    if (grid > 0x7fffffffLL) return -1;
    static bool attr_set = false;   // per instantiation
    if (!attr_set || true) {
        cudaError_t e = cudaFuncSetAttribute(nk_conv_tiled_kernel<T, KH, KW>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaFuncSetAttribute(nk_conv_tiled_kernel)");
        attr_set = true;
    }
    nk_conv_tiled_kernel<T, KH, KW><<<unsigned(grid), 256, smem, ctx->stream>>>(out, partial, I, K, p);
    int st = nk_after_launch(ctx, "nk_conv_tiled_kernel");
    if (st || splits == 1) return st;
    const int64_t plane = p.NP * int64_t(p.OH) * p.OW;
    int g = nk_grid_for(ctx, plane, 256, 8);
    nk_conv_tiled_finish_kernel<T><<<g, 256, 0, ctx->stream>>>(out, partial, p);
    return nk_after_launch(ctx, "nk_conv_tiled_finish_kernel");
}
