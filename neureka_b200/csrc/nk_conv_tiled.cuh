// Tiled direct-stencil convolution (forward, d < 0) for dense image-like calls.
//
// Shape of the work: one operand (the "image") is larger than the other (the "kernel") in the last one or two
// dims, which therefore slide (a window of KH x KW taps); every other dim is handled by the generic per-dim
// rules of the forward convolution -- it may be batch-like (kernel extent 1), summed away (equal extents,
// "channels"), an outer window (both > 1) or follow the kernel (image extent smaller) -- and is either part of
// the CTA's output coordinate or of its reduction loop.
//
// One CTA produces a TH x TW output tile for one outer output coordinate and walks the reduction loop
// ("channels") with a multi-stage shared-memory pipeline: while channel c is consumed, the (TH+KH-1) x (TW+KW-1)
// image tiles of the next channels are in flight. Two loaders exist for the same compute code:
//   * TMA  : one elected thread issues one cp.async.bulk.tensor per tile (tensor map over the image view, zero
//            fill outside the image), completion on an mbarrier -- no per-thread address arithmetic at all;
//   * LDGSTS: cp.async 16-byte (or element-wise) chunks with per-thread precomputed coordinates, for views whose
//            base or strides are not 16-byte aligned or whose rank exceeds what a tensor map can describe.
// A thread owns RH x CW outputs (CW = one 128-bit vector) and slides over the tile rows so that every
// shared-memory row segment it loads feeds up to KH output rows; the KH x KW weights of the current channel sit
// in registers. Each input byte is fetched from HBM once per tile (+ halo).
//
// Launch shapes (chosen by nk_launch_tiled from the tile count and the kernel's real occupancy):
//   * one tile per CTA, the hardware scheduling the CTAs -- a few tiles per resident CTA slot;
//   * balanced persistent walk (TMA, two sliding dims, no channel split) -- the grid is one resident wave of G CTAs.
//     Tiles are numbered with the column block fastest, then the row block, then the outer coordinate. First come
//     W = tiles / G whole waves: in wave w CTA b takes tile w * G + b, so the CTAs of a wave work side by side on one band
//     of the tensor (neighbouring column blocks of the same rows: their loads and stores form long contiguous runs in
//     DRAM). The remaining tiles -- less than one per CTA -- are not dealt whole: each is cut into groups of 8 rows, and
//     the groups of all remaining tiles, laid end to end in tile order, are dealt to the CTAs in equal contiguous ranges;
//     a range is cut into chunks of 1, 2, 4 or 8 groups that stop at tile ends, a chunk of n groups giving every warp n rows
//     (the multiply-add loop exists once per such n) and loading through the tensor map whose box is 8 n + KH - 1 rows
//     high. So the last, partial wave costs its share of a tile instead of a whole one. A CTA's chunks of that wave (at
//     most RH) are written into a table in shared memory by the producer thread during the prologue; the walk itself
//     carries no more state through the multiply-add loop than a chunk counter. The producer warp keeps loading across
//     chunk boundaries; tiles with their own weights select one of the weight sets staged at once; for one-channel
//     chunks the compute warps take tile positions from a ring the producer fills instead of decoding them (RING), or
//     run every weight set over the one image tile they hold (WLOOP, image gradients);
//   * channel split -- fewer tiles than slots and many channels: up to 8 parts of a tile form a thread-block cluster
//     and add their partial tiles through distributed shared memory; more parts go through scratch and a finish
//     kernel. Both add in part order, so the result is deterministic and the same on either path.
// The same kernel runs deconvolutions whose drain is the image-shaped tensor as a zero-padded, flipped correlation
// (padX / padY / padO / xoff of the plan).
#pragma once
#include <cuda.h>
#include <cooperative_groups.h>
#include <mutex>
#include <type_traits>
#include <vector>
#include "nk_conv_plan.h"
#include "nk_ptx.cuh"

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
    int remote_out;   // the drain lives on another GPU (stores cross NVLink)
    int persist;      // TMA family: the grid is one resident wave; whole waves of tiles, then the rest dealt in 8-row groups
    int64_t tiles_total;
    int waves;            // whole waves: in wave w CTA b takes tile w * gridDim.x + b
    int tail;             // the tiles after the whole waves are dealt in 16-row units (else whole, to the first CTAs)
    int wsets;        // persistent walk over tiles whose weights differ: weight sets staged at once (1 = same weights everywhere)
    // Weight loop (persistent walks of one-channel chunks whose outer output dims that move the kernel -- the output
    // channels of an image gradient -- touch neither the image nor the reduction): those dims are not part of the tile
    // index at all. A chunk's image tile is loaded once and every weight set is run over it in turn, each result going to
    // its own plane of the drain: wext / wos / wK are the extents, drain strides and kernel strides of those dims.
    int wloop, n_w;
    int64_t wext[NK_MAX_RANK], wos[NK_MAX_RANK], wK[NK_MAX_RANK];
    int cluster;   // channel-split CTAs of a tile form one thread-block cluster and add their tiles through shared memory
    int vec;       // LDGSTS: 16-byte global->shared copies are legal for every chunk
    int vec_out;   // 16-byte stores to the drain are legal
    int has_y;     // the second-to-last dim is the tile's row dim (else tiles are one row high)
    int tma_nd;    // TMA: dims of the tensor map (2..5)
    // Deconvolution as a padded correlation (TMA family only): tile loads start pad elements before the output
    // coordinate (the tensor map zero-fills outside the image) and the weights are staged flipped by the host's
    // choice of kernel strides. xoff shifts the tile grid left so that x0 - padX stays 16-byte aligned.
    int padX, padY, xoff;
    int padO[NK_MAX_RANK];
    int* status;   // TMA: host-mapped word, set non-zero when a bounded wait ran out
};

// One tile load: coordinates are element indices, innermost first. No multicast, local memory only.
__device__ __forceinline__ void nk_tma_load(void* smem, const CUtensorMap* map, uint64_t* bar, int nd, const int* c);
__device__ __forceinline__ void nk_tma_load5(void* smem, const CUtensorMap* map, uint64_t* bar, int nd, int c0, int c1, int c2, int c3, int c4) {
    const int c[5] = {c0, c1, c2, c3, c4};   // constant indices only below: stays in registers
    nk_tma_load(smem, map, bar, nd, c);
}
__device__ __forceinline__ void nk_tma_load(void* smem, const CUtensorMap* map, uint64_t* bar, int nd, const int* c) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem), b = (unsigned)__cvta_generic_to_shared(bar);
    unsigned long long m = reinterpret_cast<unsigned long long>(map);
    if (nd == 2)
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                     ::"r"(d), "l"(m), "r"(c[0]), "r"(c[1]), "r"(b) : "memory");
    else if (nd == 3)
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];\n"
                     ::"r"(d), "l"(m), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(b) : "memory");
    else if (nd == 4)
        asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];\n"
                     ::"r"(d), "l"(m), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(b) : "memory");
    else
        asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];\n"
                     ::"r"(d), "l"(m), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]), "r"(c[4]), "r"(b) : "memory");
}

template <class T, int KH, int KW, int RH_>
struct TiledCfg {
    static constexpr int CW = 16 / int(sizeof(T));            // outputs per thread along x = one 128-bit vector
    static constexpr int RH = RH_;                            // output rows per thread
    static constexpr int WARPS = 8;
    static constexpr int TW = 32 * CW;
    static constexpr int TH = WARPS * RH;
    static constexpr int HALO_W = ((KW - 1 + CW - 1) / CW) * CW;
    static constexpr int SW = TW + HALO_W;                    // shared row length, a multiple of CW
    static constexpr int SH = TH + KH - 1;
    static constexpr int STAGE_BYTES = ((SH * SW * int(sizeof(T)) + 127) / 128) * 128;
    static constexpr int STAGES = (STAGE_BYTES * 4 <= 64 * 1024) ? 4 : 3;
    static constexpr int NS = CW + HALO_W;                    // row-segment values a thread loads
    static constexpr int WPAD = ((KH * KW + CW - 1) / CW) * CW;
    static constexpr bool WREG = KH * KW * int(sizeof(T)) <= 400;   // weights of one channel live in registers
    static constexpr int CPR = SW / CW;                       // LDGSTS chunks per row
    static constexpr int NIT = (SH * CPR + 255) / 256;        // LDGSTS chunks per thread
    static constexpr int MAX_TAIL = 8;                        // chunks of the last, partial wave per CTA (at most RH / 2 units + 1, one each)
    static constexpr int FIXED_BYTES = 384 + MAX_TAIL * 48;
    static size_t smem_bytes(int NQ, int wsets = 1) {
        // [stages | mbarriers + abort word + tail count (128 B) | tile-info ring (256 B) | tail table (48 B per chunk) |
        //  weights | channel table (32 B per channel) | drain offset per weight set (8 B each)]
        return size_t(STAGES) * STAGE_BYTES + FIXED_BYTES + size_t(wsets) * NQ * WPAD * sizeof(T) + 16 + size_t(NQ) * 4 * sizeof(int64_t) +
               size_t(wsets) * sizeof(int64_t);
    }
};

// The tensor maps of a launch, one per rows-per-warp value r of a chunk (2, 4, 8 -> entry 0, 1, 2): a box of 8 r + KH - 1 rows.
struct TmapSet { CUtensorMap m[3]; };
__host__ __device__ constexpr int nk_tmap_slot(int r) { return r >= 8 ? 2 : (r >= 4 ? 1 : 0); }
template <int N> struct NkRows { static constexpr int value = N; };
// Variants of the persistent TMA kernel: chunks decoded by the compute warps / taken from the producer's ring / weight loop
#define NK_TILED_PLAIN 0
#define NK_TILED_RING 1
#define NK_TILED_WLOOP 2

// MODE: RING (persistent walk over short chunks only) -- the compute warps take each chunk's position from a ring the
// producer thread fills instead of decoding it themselves; WLOOP -- every chunk runs all weight sets over its one image
// tile. Compile-time switches: with the ring code merely present the long-chunk launches measured 3 % slower, and with the
// weight loop present the kernel took 168 registers instead of 93 (one CTA per SM instead of two).
// Two CTAs per SM are what the pipelined kernel is tuned for (18 warps share the issue ports; one CTA alone leaves a third
// of them idle): the state a thread carries through the multiply-add loop is kept small enough for that (the last,
// partial wave comes from a table in shared memory, not from arithmetic in registers).
// The 4-rows-per-thread F32 kernels fit three CTAs per SM (three stages of 19 KB each) if their registers allow it: 72
// instead of the 92-94 the compiler takes by itself, without spills (measured 2-6 % faster on short images and their
// gradients). Every other instantiation passes 0 = no statement: an explicit 1 makes the compiler spend registers freely
// (the 8-row F32 5x5 kernel went from 96 to 111 and lost its second CTA per SM: 0.99 -> 1.22 ms on config 5).
template <class T, int KH, int KW, int RH, bool TMA, int MODE = NK_TILED_PLAIN>
__global__ void __launch_bounds__(TMA ? 288 : 256, (TMA && RH == 4 && sizeof(T) == 4) ? 3 : 0) nk_conv_tiled_kernel(T* __restrict__ out, T* __restrict__ partial,
                                                            const T* __restrict__ I, const T* __restrict__ K,
                                                            const TiledPlan p, const __grid_constant__ TmapSet tmaps) {
    using C = TiledCfg<T, KH, KW, RH>;
    constexpr int CW = C::CW, TW = C::TW, TH = C::TH, SW = C::SW, SH = C::SH, STAGES = C::STAGES, NS = C::NS, WPAD = C::WPAD;
    constexpr bool RING = MODE == NK_TILED_RING, WLOOP = MODE == NK_TILED_WLOOP;
    extern __shared__ __align__(128) unsigned char nk_smem[];
    unsigned char* stage_base = nk_smem;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(nk_smem + size_t(STAGES) * C::STAGE_BYTES);
    // Where a chunk lives, two int4: (x0, y0, weight set, first row below the chunk) and (drain base low, high, rows per
    // warp, 0). Persistent walk, RING: the producer thread publishes every chunk in a ring of STAGES + 1 such entries and
    // the compute warps pick an entry up after the chunk's first load landed.
    int4* tinfo = reinterpret_cast<int4*>(nk_smem + size_t(STAGES) * C::STAGE_BYTES + 128);
    // Persistent walk: the chunks of the last, partial wave of this CTA, written once in the prologue: entries of three
    // int4, the two above and the chunk's tensor-map coordinates 1..4 without their channel part.
    int4* tail_tab = reinterpret_cast<int4*>(nk_smem + size_t(STAGES) * C::STAGE_BYTES + 384);
    T* wsm = reinterpret_cast<T*>(nk_smem + size_t(STAGES) * C::STAGE_BYTES + C::FIXED_BYTES);
    // channel table, 32 bytes per channel: image offset, kernel offset, then the tile's tensor-map coordinates 1..4
    // (everything but x) ready for the producer thread -- it runs on the same issue port as two compute warps per
    // CTA, and every instruction it spends per tile is taken from them
    int64_t* ctab = reinterpret_cast<int64_t*>((reinterpret_cast<uintptr_t>(wsm + size_t(p.wsets) * p.NQ * WPAD) + 15) & ~uintptr_t(15));

    int64_t* wofs = ctab + size_t(p.NQ) * 4;   // weight loop: where weight set ws stores, relative to the chunk's drain base

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

    // ---- which tile / outer coordinate / channel range ----------------------------------------------------------
    // One tile per CTA (the parts of a channel split are neighbours: one cluster), or -- persistent -- whole tiles
    // blockIdx.x, blockIdx.x + gridDim.x, ... for p.waves steps and then the CTA's chunks of the last, partial wave, with the
    // load pipeline running on across chunk boundaries.
    const int split = p.persist ? 0 : int(blockIdx.x % unsigned(p.splits));
    // whole tiles of this CTA: p.waves, and one more for the first CTAs when the last, partial wave is dealt in whole tiles too
    const int my_waves = p.waves + ((p.persist && !p.tail && int64_t(blockIdx.x) < p.tiles_total - int64_t(p.waves) * gridDim.x) ? 1 : 0);
    const int64_t tile_first = p.persist ? (my_waves > 0 ? int64_t(blockIdx.x) : 0) : int64_t(blockIdx.x / unsigned(p.splits));
    const int64_t tile_step = gridDim.x;
    int64_t baseI, baseK, baseO;
    int pidx[NK_TILED_MAX_OUTER];
    int x0, y0;
    int rh_cur = RH;        // rows per warp of the chunk / tile this thread stands on
    int y_end = p.OH;       // first row below it
    int wset = 0;   // which of the staged weight sets the current tile uses (outer output dims that move the kernel)
    // Takes a tile index apart with divisions (once per thread, and once per tile of long tiles; the producer thread of a
    // persistent CTA steps on digit by digit instead, see below).
    auto tile_set = [&](int64_t tile) {
        const int tx = int(tile % p.tilesX); tile /= p.tilesX;
        const int ty = int(tile % p.tilesY); tile /= p.tilesY;
        baseI = p.bI; baseK = p.bK; baseO = p.bO;
        int64_t rem = tile;
        int ws = 0, wm = 1;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            const int idx = int(rem % p.oext[k]);
            rem /= p.oext[k];
            baseI += idx * p.pI[k]; baseK += idx * p.pK[k]; baseO += idx * p.os[k];
            pidx[k] = p.pI[k] != 0 ? idx : 0;   // the image index follows the output index only where pI != 0
            if (p.pK[k] != 0) { ws += idx * wm; wm *= int(p.oext[k]); }
        }
        wset = p.wsets > 1 ? ws : 0;
        x0 = tx * TW - p.xoff;
        y0 = ty * TH;
    };
    // puts the thread on a chunk described by two int4 (ring entry or the head of a table entry)
    auto place = [&](const int4 a, const int4 b) {
        x0 = a.x; y0 = a.y; wset = a.z; y_end = a.w;
        baseO = (int64_t(b.y) << 32) | int64_t(unsigned(b.x));
        rh_cur = b.z;
    };
    tile_set(tile_first);
    const int64_t pflat = tile_first / (int64_t(p.tilesX) * p.tilesY);   // used by the two-pass split path (one tile per CTA)
    const int cper = (p.NQ + p.splits - 1) / p.splits;
    const int c_begin = split * cper;
    const int c_end = (c_begin + cper < p.NQ) ? c_begin + cper : p.NQ;

    // TMA family: warps 0..7 compute, warp 8 feeds the pipeline. full[s] completes when the tile has landed
    // (1 arrival + the tile's bytes), empty[s] when all 8 compute warps have finished reading stage s.
    uint64_t* full_bar = mbar;
    uint64_t* empty_bar = mbar + STAGES;
    volatile int* abort_word = reinterpret_cast<volatile int*>(mbar + 2 * STAGES);
    int* n_tail_word = reinterpret_cast<int*>(mbar + 2 * STAGES) + 1;   // entries of tail_tab
    const int n_it = c_end - c_begin;
    int issued = 0;                            // tiles requested so far (producer thread)
    // Tensor-map coordinates 1..4 of a tile load (coordinate 0 is x0 - padX): a part that depends on the channel only
    // (kept in the channel table) plus a part that depends on the output tile only.
    auto chan_coords = [&](int c, int* cc) {
        cc[0] = cc[1] = cc[2] = cc[3] = 0;
        int n = 0;
        if (p.has_y) cc[n++] = -p.padY;
        int rem = c;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            const int q = rem % int(p.qext[k]);
            rem /= int(p.qext[k]);
            if (n < 4) cc[n] = q - p.padO[k];
            n++;
        }
    };
    auto tile_coords = [&]() -> int4 {   // of the tile this thread currently stands on
        int b[4] = {0, 0, 0, 0};
        int n = 0;
        if (p.has_y) b[n++] = y0;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            if (n < 4) b[n] = pidx[k];
            n++;
        }
        return make_int4(b[0], b[1], b[2], b[3]);
    };
    // Bytes and tensor map of a tile load for a chunk of rh rows per warp: worked out once per chunk, not per load (every
    // instruction of the producer thread is taken from the compute warps it shares an issue port with).
    auto chunk_bytes = [&](int rh) -> unsigned {
        // without a row dim in the map the box is a single row; the other tile rows are never stored from
        return unsigned((p.has_y ? 8 * rh + KH - 1 : 1) * SW * sizeof(T));
    };
    auto tma_fire = [&](int stage, unsigned bytes, const CUtensorMap* map, int c1, int c2, int c3, int c4) {
        nk_mbar_expect_tx(&full_bar[stage], bytes);
        nk_tma_load5(stage_base + size_t(stage) * C::STAGE_BYTES, map, &full_bar[stage], p.tma_nd, x0 - p.padX, c1, c2, c3, c4);
        issued++;
    };
    if (TMA && tid == 256) {
        // the producer thread sets the barriers up and requests the first tiles right away, so that they travel
        // while the other warps stage the weights; everybody else meets the barriers only after the __syncthreads below
        for (int s = 0; s < STAGES; s++) { nk_mbar_init(&full_bar[s], 1); nk_mbar_init(&empty_bar[s], 8); }
        *abort_word = 0;
        nk_fence_barrier_init();
        nk_fence_proxy_async();
        auto first_loads = [&](const int4 tb) {   // of the chunk this thread stands on
            for (int it = 0; it < STAGES && it < n_it; it++) {
                int cc[4];
                chan_coords(c_begin + it, cc);
                tma_fire(it, chunk_bytes(rh_cur), &tmaps.m[nk_tmap_slot(rh_cur)], cc[0] + tb.x, cc[1] + tb.y, cc[2] + tb.z, cc[3] + tb.w);
            }
        };
        if (!p.persist) {
            first_loads(tile_coords());
        } else {
            if (my_waves > 0) first_loads(tile_coords());
            // The last, partial wave (p.tail): the tiles after the whole waves are cut into units of 16 rows (RH / 2 per tile) and
            // the units, laid end to end in tile order, dealt to the CTAs in equal contiguous ranges -- less than one tile's
            // worth each. A range is cut into chunks of 1, 2 or 4 units (2, 4, 8 rows per warp: the multiply-add loop
            // exists for those) that stop at tile ends; chunks entirely below the image's last row are dropped.
            constexpr int UPT = RH / 2;
            const int64_t G = gridDim.x;
            const int64_t tail_first = int64_t(p.waves) * G;
            const int64_t tail_units = p.tail ? (p.tiles_total - tail_first) * UPT : 0;
            int64_t q = (int64_t(blockIdx.x) * tail_units) / G;
            const int64_t q_hi = (int64_t(blockIdx.x + 1) * tail_units) / G;
            int nt = 0;
            while (q < q_hi && nt < C::MAX_TAIL) {
                const int64_t t = q / UPT;
                const int u0 = int(q - t * UPT);
                int n = UPT - u0;
                if (int64_t(n) > q_hi - q) n = int(q_hi - q);
                n = n >= 4 ? 4 : n >= 2 ? 2 : 1;
                q += n;
                tile_set(tail_first + t);
                y0 += u0 * 16;
                int h = p.OH - y0;
                if (h <= 0) continue;
                if (h > n * 16) h = n * 16;
                const int r = (h + 7) >> 3;   // rows per warp: the next of 2, 4, 8 (rows below y0 + h are not stored)
                int4* e = tail_tab + 3 * nt;
                e[0] = make_int4(x0, y0, wset, y0 + h);
                e[1] = make_int4(int(unsigned(baseO & 0xffffffffLL)), int(baseO >> 32), r > 4 ? 8 : r > 2 ? 4 : 2, 0);
                e[2] = tile_coords();
                nt++;
            }
            *n_tail_word = nt;
            if (my_waves > 0) {
                tile_set(tile_first);   // back on the first whole tile
            } else if (nt > 0) {
                place(tail_tab[0], tail_tab[1]);
                first_loads(tail_tab[2]);
            }
        }
    }

    // ---- stage the channel table and this CTA's weights ---------------------------------------------------------
    for (int c = c_begin + tid; c < c_end; c += blockDim.x) {
        int rem = c;
        int64_t oi = 0, ok = 0;
        for (int k = p.n_outer - 1; k >= 0; k--) {
            int q = rem % int(p.qext[k]);
            rem /= int(p.qext[k]);
            oi += q * p.qI[k]; ok += q * p.qK[k];
        }
        ctab[c * 4 + 0] = oi;
        ctab[c * 4 + 1] = ok;
        int cc[4];
        chan_coords(c, cc);
        *reinterpret_cast<int4*>(&ctab[c * 4 + 2]) = make_int4(cc[0], cc[1], cc[2], cc[3]);
    }
    __syncthreads();
    for (int e = tid; e < p.wsets * (c_end - c_begin) * WPAD; e += blockDim.x) {
        const int per_set = (c_end - c_begin) * WPAD;
        const int ws = e / per_set, r = e - ws * per_set;
        const int c = c_begin + r / WPAD, t = r % WPAD;
        int64_t kb = baseK;   // one set: the weights of this CTA's (only, or every) tile
        if (p.wloop) {        // the sets of the weight loop: set ws belongs to index ws of the dims taken out of the tile index
            kb = p.bK;
            int rem = ws;
            for (int k = p.n_w - 1; k >= 0; k--) { kb += int64_t(rem % int(p.wext[k])) * p.wK[k]; rem /= int(p.wext[k]); }
        } else if (p.wsets > 1) {    // several: set ws belongs to the outer output indices that tile_set() folds into ws
            kb = p.bK;
            int rem = ws;
            for (int k = p.n_outer - 1; k >= 0; k--)
                if (p.pK[k] != 0) { kb += int64_t(rem % int(p.oext[k])) * p.pK[k]; rem /= int(p.oext[k]); }
        }
        T v = 0;
        if (t < KH * KW) v = K[kb + ctab[c * 4 + 1] + (t / KW) * p.sKy + (t % KW) * p.sKx];
        wsm[(size_t(ws) * p.NQ + c) * WPAD + t] = v;
    }

    if (p.wloop) {
        for (int ws = tid; ws < p.wsets; ws += blockDim.x) {
            int rem = ws;
            int64_t o = 0;
            for (int k = p.n_w - 1; k >= 0; k--) { o += int64_t(rem % int(p.wext[k])) * p.wos[k]; rem /= int(p.wext[k]); }
            wofs[ws] = o;
        }
    }

    // ---- loaders ------------------------------------------------------------------------------------------------
    // LDGSTS: the chunk coordinates of a thread do not depend on the channel -- compute them once
    int l_soff[TMA ? 1 : C::NIT], l_bytes[TMA ? 1 : C::NIT];
    int64_t l_goff[TMA ? 1 : C::NIT];
    if (!TMA) {
#pragma unroll
        for (int it = 0; it < C::NIT; it++) {
            const int id = tid + it * 256;
            const int row = id / C::CPR, col = (id - row * C::CPR) * CW;
            const int gy = y0 + row, gx = x0 + col;
            int valid = (id < SH * C::CPR && gy < p.IH) ? (p.IW - gx) : 0;
            valid = valid < 0 ? 0 : (valid > CW ? CW : valid);
            l_soff[it] = (id < SH * C::CPR) ? (row * SW + col) : -1;
            l_bytes[it] = valid * int(sizeof(T));
            l_goff[it] = valid > 0 ? (int64_t(gy) * p.sIy + gx) : 0;
        }
    }
    auto ldgsts_stage = [&](int stage, int c) {
        T* dst = reinterpret_cast<T*>(stage_base + size_t(stage) * C::STAGE_BYTES);
        const T* src = I + baseI + ctab[c * 4 + 0];
#pragma unroll
        for (int it = 0; it < C::NIT; it++) {
            if (l_soff[it] < 0) continue;
            T* s = dst + l_soff[it];
            const T* g = src + l_goff[it];
            if (p.vec) {
                nk_cp_async_16(s, g, l_bytes[it]);
            } else {
#pragma unroll
                for (int e = 0; e < CW; e++) {
                    const int ok = (e * int(sizeof(T)) < l_bytes[it]) ? int(sizeof(T)) : 0;
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

    __syncthreads();   // weights + table + barrier init visible

    // One channel's worth of multiply-adds for this thread, RHC rows per warp (tile rows warp*RHC .. +RHC, columns
    // lane*CW .. +CW). The order of the additions into one output does not depend on RHC: channel, then ky, then kx.
    auto consume = [&](auto rows_tag, const unsigned char* box, int c) {
        constexpr int RHC = decltype(rows_tag)::value;
        const T* tile = reinterpret_cast<const T*>(box) + (warp * RHC) * SW + lane * CW;
        const T* wc = wsm + (size_t(wset) * p.NQ + c) * WPAD;
        T w[C::WREG ? WPAD : CW];
        if (C::WREG) {
#pragma unroll
            for (int v = 0; v < WPAD / CW; v++) {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(&w[v * CW]) = *reinterpret_cast<const float4*>(wc + v * CW);
                else *reinterpret_cast<double2*>(&w[v * CW]) = *reinterpret_cast<const double2*>(wc + v * CW);
            }
        }
#pragma unroll
        for (int j = 0; j < RHC + KH - 1; j++) {
            T seg[NS];
#pragma unroll
            for (int v = 0; v < NS / CW; v++) {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(&seg[v * CW]) = *reinterpret_cast<const float4*>(tile + j * SW + v * CW);
                else *reinterpret_cast<double2*>(&seg[v * CW]) = *reinterpret_cast<const double2*>(tile + j * SW + v * CW);
            }
#pragma unroll
            for (int i = 0; i < RHC; i++) {
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
    };
    // Stores this thread's results of the tile / chunk the thread currently stands on (rh_cur rows per warp, rows below
    // y_end only): into the drain, or -- two-pass channel split -- into this part's plane of the scratch buffer.
    auto store_tile = [&](int64_t plane_off = 0) {
        const int ox = x0 + lane * CW;
#pragma unroll
        for (int i = 0; i < RH; i++) {
            const int oy = y0 + warp * rh_cur + i;
            if (i >= rh_cur || oy >= y_end || ox >= p.OW || ox + CW <= 0) continue;
            T* dst;
            bool vec_ok;
            if (p.splits == 1) {
                dst = out + baseO + plane_off + int64_t(oy) * p.sOy + ox;
                vec_ok = p.vec_out != 0;
            } else {
                dst = partial + ((int64_t(split) * p.NP + pflat) * p.OH + oy) * int64_t(p.OW) + ox;
                vec_ok = (p.OW % CW) == 0;
            }
            if (vec_ok && ox >= 0 && ox + CW <= p.OW) {
                if (sizeof(T) == 4) *reinterpret_cast<float4*>(dst) = *reinterpret_cast<float4*>(&acc[i][0]);
                else *reinterpret_cast<double2*>(dst) = *reinterpret_cast<double2*>(&acc[i][0]);
            } else {
#pragma unroll
                for (int x = 0; x < CW; x++)
                    if (ox + x >= 0 && ox + x < p.OW) dst[x] = acc[i][x];
            }
        }
    };

    bool aborted = false;
    if (TMA) {
        // Every wait below is bounded; whoever runs out raises the CTA's abort word (and the host-visible status),
        // everybody else notices it while polling, and the CTA leaves without storing anything more.
        auto wait_or_abort = [&](uint64_t* bar, unsigned parity) -> bool {
            const int r = nk_mbar_wait_bounded(bar, parity, NK_WAIT_LIMIT_NS, abort_word);
            if (r < 0) {
                *abort_word = 1;
                if (p.status) atomicExch(p.status, 1);
            }
            return r > 0;
        };
        // chunks of this CTA's walk: the whole tiles, then the entries of the table
        const int n_chunks = p.persist ? my_waves + *n_tail_word : 1;
        if (warp == 8) {
            if (lane == 0 && n_chunks > 0) {
                // `issued` counts tile loads over the CTA's whole life: load g uses stage g % STAGES in round g / STAGES.
                // A tile index is a mixed-radix number (tx | ty | outer output indices, last outer dim fastest); a whole
                // wave adds gridDim.x to it, digit by digit with carry -- a few adds and compares per tile, no division.
                // Everything the step needs sits in registers under compile-time indices (j counts the outer dims from the
                // last one): the producer's time per tile bounds short tiles. Chunks of the last, partial wave come from
                // the table.
                constexpr int NO = NK_TILED_MAX_OUTER, NDIG = 2 + NO;
                int dg[NDIG], sg[NDIG], rx[NDIG], wmj[NO];
                long long osj[NO];
                bool foli[NO];
                if (p.persist && my_waves > 1) {
                    int64_t t = tile_first, st = tile_step;
#pragma unroll
                    for (int i = 0; i < NDIG; i++) {
                        rx[i] = i == 0 ? p.tilesX : i == 1 ? p.tilesY : ((i - 2) < p.n_outer ? int(p.oext[p.n_outer - 1 - (i - 2)]) : 1);
                        dg[i] = int(t % rx[i]); t /= rx[i];
                        sg[i] = int(st % rx[i]); st /= rx[i];
                    }
                    int wm = 1;
#pragma unroll
                    for (int j = 0; j < NO; j++) {
                        const bool on = j < p.n_outer;
                        const int k = on ? p.n_outer - 1 - j : 0;
                        osj[j] = on ? p.os[k] : 0;
                        foli[j] = on && p.pI[k] != 0;
                        const bool moves_kernel = on && p.pK[k] != 0;
                        wmj[j] = moves_kernel ? wm : 0;
                        if (moves_kernel) wm *= int(p.oext[k]);
                    }
                }
                bool ok = true;
                int chunk_no = 0;
                bool announce = false;      // a new chunk's info still has to go into the ring (after the stage came free)
                int4 tb = p.persist && my_waves == 0 ? tail_tab[2] : tile_coords();
                unsigned cur_bytes = chunk_bytes(rh_cur);
                const CUtensorMap* cur_map = &tmaps.m[nk_tmap_slot(rh_cur)];
                int c = c_begin + issued;   // the first loads of the first chunk were requested in the prologue
                // stage and round parity of load number `issued`, counted along instead of divided out (STAGES may be 3)
                int pstage = issued == STAGES ? 0 : issued;
                unsigned pround = issued == STAGES ? 1u : 0u;
                while (ok) {
                    if (c >= c_end) {
                        chunk_no++;
                        if (chunk_no >= n_chunks) break;
                        if (chunk_no < my_waves) {
                            int carry = 0;
#pragma unroll
                            for (int i = 0; i < NDIG; i++) {
                                const int v = dg[i] + sg[i] + carry;
                                carry = v >= rx[i] ? 1 : 0;
                                dg[i] = v - (carry ? rx[i] : 0);
                            }
                            baseO = p.bO;
                            int ws = 0, P[NO];
#pragma unroll
                            for (int j = 0; j < NO; j++) {
                                baseO += dg[2 + j] * osj[j];
                                P[j] = foli[j] ? dg[2 + j] : 0;
                                ws += dg[2 + j] * wmj[j];
                            }
                            wset = p.wsets > 1 ? ws : 0;
                            x0 = dg[0] * TW - p.xoff;
                            y0 = dg[1] * TH;
                            tb = make_int4(y0, P[0], P[1], P[2]);   // persistent walks always have a row dim: coordinate 1 is y
                        } else {
                            const int4* e = tail_tab + 3 * (chunk_no - my_waves);
                            place(e[0], e[1]);
                            tb = e[2];
                            cur_bytes = chunk_bytes(rh_cur);
                            cur_map = &tmaps.m[nk_tmap_slot(rh_cur)];
                        }
                        c = c_begin;
                        announce = true;
                    }
                    const int stage = pstage;
                    if (issued >= STAGES) ok = wait_or_abort(&empty_bar[stage], (pround & 1u) ^ 1u);
                    if (++pstage == STAGES) { pstage = 0; pround++; }
                    if (ok) {
                        if (RING && announce) {
                            // every compute warp is past the chunk whose entry this overwrites (ring of STAGES + 1, at least
                            // one load per chunk, and the wait above); the arrive inside tma_fire publishes the stores
                            int4* e = tinfo + 2 * (chunk_no % (STAGES + 1));
                            e[0] = make_int4(x0, y0, wset, y_end);
                            e[1] = make_int4(int(unsigned(baseO & 0xffffffffLL)), int(baseO >> 32), rh_cur, 0);
                            announce = false;
                        }
                        const int4 cc = *reinterpret_cast<const int4*>(&ctab[c * 4 + 2]);
                        tma_fire(stage, cur_bytes, cur_map, cc.x + tb.x, cc.y + tb.y, cc.z + tb.z, cc.w + tb.w);
                    }
                    c++;
                }
                if (!ok || *abort_word) {
                    // requested copies may still be landing in this CTA's shared memory: wait for the last ones (bounded)
                    for (int j = (issued > STAGES ? issued - STAGES : 0); j < issued; j++) {
                        nk_mbar_wait_bounded(&full_bar[j % STAGES], unsigned(j / STAGES) & 1u, NK_WAIT_LIMIT_NS, nullptr);
                    }
                }
            }
        } else {
            int cstage = 0;        // stage and round parity of the next load to consume (same numbering as the producer's)
            unsigned cpar = 0;
            bool ok = true;
            // the channel loop of one chunk, specialised on the rows per warp: the choice sits outside the loop, so the
            // loop body is straight-line code the compiler can schedule across iterations, as for a fixed tile height
            auto run_chunk = [&](auto rows_tag) {
                if constexpr (WLOOP) {
                    // one image tile (a single channel), every weight set in turn: multiply-adds, store, clear. The
                    // stage goes back to the producer after the last set's multiply-adds.
                    constexpr int RHC = decltype(rows_tag)::value;
                    const int stage = cstage;
                    if (!wait_or_abort(&full_bar[stage], cpar)) { ok = false; return; }
                    // where this thread's rows go does not depend on the weight set: worked out once per chunk
                    const int ox = x0 + lane * CW;
                    const bool fast = p.vec_out != 0 && ox >= 0 && ox + CW <= p.OW;   // whole 16-byte stores
                    T* const dst0 = out + baseO + int64_t(y0 + warp * RHC) * p.sOy + ox;
                    const int rows_ok = y_end - (y0 + warp * RHC);                     // rows of this thread inside the chunk
                    for (int ws = 0; ws < p.wsets; ws++) {
                        wset = ws;
                        // the tile's address is made opaque per weight set: otherwise the compiler keeps the whole tile in
                        // registers across the loop (168 of them, one CTA per SM: measured 20 % slower)
                        int st = stage;
                        asm volatile("" : "+r"(st));
                        consume(rows_tag, stage_base + size_t(st) * C::STAGE_BYTES, c_begin);
                        if (ws + 1 == p.wsets) {
                            __syncwarp();
                            if (lane == 0) nk_mbar_arrive(&empty_bar[stage]);
                        }
                        if (fast) {
                            T* d = dst0 + wofs[ws];
#pragma unroll
                            for (int i = 0; i < RHC; i++) {
                                if (i < rows_ok) {
                                    if (sizeof(T) == 4) *reinterpret_cast<float4*>(d) = *reinterpret_cast<float4*>(&acc[i][0]);
                                    else *reinterpret_cast<double2*>(d) = *reinterpret_cast<double2*>(&acc[i][0]);
                                }
                                d += p.sOy;
                            }
                        } else {
                            store_tile(wofs[ws]);
                        }
#pragma unroll
                        for (int i = 0; i < RH; i++)
#pragma unroll
                            for (int x = 0; x < CW; x++) acc[i][x] = T(0);
                    }
                    if (++cstage == STAGES) { cstage = 0; cpar ^= 1u; }
                } else {
                    for (int c = c_begin; c < c_end; c++) {
                        const int stage = cstage;
                        if (!wait_or_abort(&full_bar[stage], cpar)) { ok = false; break; }
                        consume(rows_tag, stage_base + size_t(stage) * C::STAGE_BYTES, c);
                        __syncwarp();
                        if (lane == 0) nk_mbar_arrive(&empty_bar[stage]);
                        if (++cstage == STAGES) { cstage = 0; cpar ^= 1u; }
                    }
                }
            };
            for (int chunk_no = 0; chunk_no < n_chunks; chunk_no++) {
                if (chunk_no >= my_waves && p.persist) {
                    // a chunk of the last, partial wave: 2, 4 or RH rows per warp
                    const int4* e = tail_tab + 3 * (chunk_no - my_waves);
                    place(e[0], e[1]);
                } else if (chunk_no > 0) {
                    if (RING) {
                        // where this tile lives: published by the producer before the tile's first load, so wait for that
                        // load (the loop below finds it complete) and pick the entry up
                        if (!wait_or_abort(&full_bar[cstage], cpar)) { ok = false; break; }
                        const int4* e = tinfo + 2 * (chunk_no % (STAGES + 1));
                        place(e[0], e[1]);
                    } else {
                        tile_set(tile_first + chunk_no * tile_step);   // long tiles: a dozen divisions per tile do not matter
                    }
                }
                if (rh_cur == RH) run_chunk(NkRows<RH>{});
                else if (rh_cur == 2) run_chunk(NkRows<2>{});
                else { if constexpr (RH > 4) run_chunk(NkRows<4>{}); }
                if (!ok || !p.persist) break;   // one tile per CTA: its epilogue follows below
                if constexpr (!WLOOP) {         // (the weight loop stores every set's result itself)
                    store_tile();
#pragma unroll
                    for (int i = 0; i < RH; i++)
#pragma unroll
                        for (int x = 0; x < CW; x++) acc[i][x] = T(0);
                }
            }
        }
        __syncthreads();
        if (p.persist) return;   // every chunk was stored on the way
        if (*abort_word) {
            if (!p.cluster) return;
            aborted = true;   // the cluster's barriers below still have to be met; the host reports the time-out
        }
        if (warp == 8 && !p.cluster) return;   // the producer warp owns no outputs
    } else {
#pragma unroll
        for (int s = 0; s < STAGES - 1; s++) {
            if (s < n_it) ldgsts_stage(s, c_begin + s);
            nk_cp_async_commit();
        }
        for (int it = 0; it < n_it; it++) {
            nk_cp_async_wait<STAGES - 2>();
            __syncthreads();   // tile `it` has landed for everyone; everyone is done reading the stage refilled below
            const int nxt = it + STAGES - 1;
            if (nxt < n_it) ldgsts_stage(nxt % STAGES, c_begin + nxt);
            nk_cp_async_commit();
            consume(NkRows<RH>{}, stage_base + size_t(it % STAGES) * C::STAGE_BYTES, c_begin + it);
        }
        nk_cp_async_wait<0>();
    }

    // ---- epilogue of a one-tile CTA ---------------------------------------------------------------------------------
    if (p.cluster) {
        // The p.splits CTAs of this tile are one cluster (rank == split). Each leaves its partial tile in its own
        // shared memory; then CTA r adds slice r of the tile over all ranks, in rank order (the same order as the
        // two-pass path, so both give the same bits), reading the peers' tiles through distributed shared memory.
        namespace cg = cooperative_groups;
        cg::cluster_group cl = cg::this_cluster();
        using V = typename std::conditional<sizeof(T) == 4, float4, double2>::type;
        T* red = reinterpret_cast<T*>(stage_base);   // every tile load has been consumed: the ring is free
        __syncthreads();
        if (warp < 8 && !aborted) {
#pragma unroll
            for (int i = 0; i < RH; i++)
                *reinterpret_cast<V*>(red + ((warp * RH + i) * TW + lane * CW)) = *reinterpret_cast<V*>(&acc[i][0]);
        }
        cl.sync();
        constexpr int VPR = TW / CW, NV = TH * VPR;
        const int per = (NV + p.splits - 1) / p.splits;
        const int v_end = ((split + 1) * per < NV) ? (split + 1) * per : NV;
        const T* peer[8];
#pragma unroll
        for (int s = 0; s < 8; s++) peer[s] = cl.map_shared_rank(red, s < p.splits ? s : 0);
        for (int v = split * per + tid; v < v_end && !aborted; v += blockDim.x) {
            // all parts are fetched before the first addition: the remote reads overlap instead of queueing up
            T part[8][CW];
#pragma unroll
            for (int s = 0; s < 8; s++)
                if (s < p.splits) *reinterpret_cast<V*>(part[s]) = *reinterpret_cast<const V*>(peer[s] + size_t(v) * CW);
            T sum[CW];
#pragma unroll
            for (int x = 0; x < CW; x++) sum[x] = T(0);
#pragma unroll
            for (int s = 0; s < 8; s++)
                if (s < p.splits) {
#pragma unroll
                    for (int x = 0; x < CW; x++) sum[x] += part[s][x];
                }
            const int oy = y0 + v / VPR, ox = x0 + (v % VPR) * CW;
            if (oy >= p.OH || ox >= p.OW || ox + CW <= 0) continue;
            T* dst = out + baseO + int64_t(oy) * p.sOy + ox;
            if (p.vec_out && ox >= 0 && ox + CW <= p.OW) {
                *reinterpret_cast<V*>(dst) = *reinterpret_cast<V*>(sum);
            } else {
#pragma unroll
                for (int x = 0; x < CW; x++)
                    if (ox + x >= 0 && ox + x < p.OW) dst[x] = sum[x];
            }
        }
        cl.sync();   // nobody leaves while a peer may still be reading its tile
        return;
    }
    store_tile();
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

// Host side of a TMA launch: everything needed to encode the tensor map of the image view.
struct TmaImage {
    const void* base;            // address of element (0,..,0) of the view
    int nd;                      // dims, innermost first
    uint64_t dims[5];
    uint64_t strides_bytes[5];   // strides_bytes[0] is the element size
};
int nk_tma_encode(nk_ctx* ctx, int dtype, const TmaImage& img, int box_w, int box_h, bool has_y, CUtensorMap* out);

// CTAs of `kern` resident per SM with `smem` bytes of dynamic shared memory, after allowing the kernel that much. Both runtime
// calls are made once per (kernel, device, size): they cost microseconds each, which is most of a launch for problems that
// live in L2.
inline int nk_tiled_occupancy(nk_ctx* ctx, const void* kern, int threads, size_t smem, int* per_sm) {
    struct Entry { const void* kern; int device; size_t smem; int per_sm; };   // per_sm < 0: the largest size allowed so far
    static std::mutex mu;
    static std::vector<Entry> cache;
    std::lock_guard<std::mutex> lock(mu);
    Entry* allowed = nullptr;
    for (Entry& e : cache) {
        if (e.kern != kern || e.device != ctx->device) continue;
        if (e.per_sm < 0) allowed = &e;
        else if (e.smem == smem) { *per_sm = e.per_sm; return 0; }
    }
    if (!allowed || allowed->smem < smem) {   // the attribute is a maximum: only ever raised
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaFuncSetAttribute(nk_conv_tiled_kernel)");
        if (allowed) allowed->smem = smem;
        else cache.push_back(Entry{kern, ctx->device, smem, -1});
    }
    int n = 1;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, threads, smem) != cudaSuccess || n < 1) {
        cudaGetLastError();
        n = 1;
    }
    *per_sm = n;
    cache.push_back(Entry{kern, ctx->device, smem, n});
    return 0;
}

template <class T, int KH, int KW, int RH, bool TMA>
int nk_launch_tiled(nk_ctx* ctx, T* out, const T* I, const T* K, TiledPlan& p, const TmaImage* img) {
    using C = TiledCfg<T, KH, KW, RH>;
    p.tilesX = (p.OW + p.xoff + C::TW - 1) / C::TW;
    p.tilesY = (p.OH + C::TH - 1) / C::TH;
    const int64_t tiles = int64_t(p.tilesX) * p.tilesY * p.NP;
    // Outer output dims that move the kernel operand (each output channel of an image gradient has its own weights):
    // a persistent walk needs all those weight sets in shared memory at once -- fine while they are small.
    int64_t wsets = 1;
    for (int k = 0; k < p.n_outer; k++)
        if (p.pK[k] != 0) wsets *= p.oext[k];
    if (p.wloop)   // those dims were taken out of the tile index by the caller: every chunk runs all of their weight sets
        for (int k = 0; k < p.n_w; k++) wsets *= p.wext[k];
    const bool sets_fit = wsets == 1 || (TMA && wsets * int64_t(p.NQ) * C::WPAD * int64_t(sizeof(T)) <= 16384);
    size_t smem = 0;
    int64_t slots = 0;
    int splits = 1;
    // shared memory, occupancy and channel split for a launch that stages `w` weight sets
    auto configure = [&](int w) -> int {
        smem = C::smem_bytes(p.NQ, w);
        if (smem > size_t(ctx->prop.sharedMemPerBlockOptin)) return -1;   // caller falls back to another family
        int per_sm = 1;
        const int ost = nk_tiled_occupancy(ctx, reinterpret_cast<const void*>(nk_conv_tiled_kernel<T, KH, KW, RH, TMA>), TMA ? 288 : 256, smem, &per_sm);
        if (ost) return ost;
        slots = int64_t(ctx->prop.multiProcessorCount) * per_sm;
        // channel split: only when the tiles alone cannot fill the machine and each part keeps >= 4 channels; the
        // CTA count stays within one resident wave (a second, nearly empty wave would double the time)
        splits = 1;
        if (tiles < slots && p.NQ >= 8) {
            splits = int(slots / tiles);
            if (splits > p.NQ / 4) splits = p.NQ / 4;
            if (splits > 32) splits = 32;
            if (splits < 1) splits = 1;
        }
        return 0;
    };
    p.wsets = (sets_fit && wsets > 1) ? int(wsets) : 1;
    int cst = configure(p.wsets);
    // The balanced persistent walk: a tensor map with a row dim, no channel split, and the same weights for every
    // strip or all weight sets resident at once.
    auto balanced = [&]() { return TMA && p.has_y && splits == 1 && (wsets == 1 || p.wsets > 1); };
    if (p.wloop && (cst != 0 || !sets_fit || !balanced())) return -1;   // the caller plans the call again without the weight loop
    if (cst == 0 && p.wsets > 1 && !balanced()) {   // no persistent walk after all: one set per CTA
        p.wsets = 1;
        cst = configure(1);
    }
    if (cst) return cst;
    p.splits = splits;
    p.cluster = 0;
    p.persist = 0;
    p.tiles_total = tiles;
    p.waves = 0;
    p.tail = 0;
    TmapSet tmaps;
    memset(&tmaps, 0, sizeof(tmaps));
    bool ring = false;
    int64_t grid = tiles * splits;
    if (TMA) {
        if (C::SW > 256 || C::SH > 256) return -1;
        p.persist = balanced() ? 1 : 0;
        // Few tiles per resident CTA slot and the same weights everywhere: one tile per CTA, dealt by the hardware as CTAs
        // retire, balances better than any fixed assignment and skips the walk's set-up. Measured on B200 (F32 5x5, 32
        // channels; persistent / one tile per CTA): 1.7 tiles per slot 0.162 / 0.155 ms, 3.5: 0.288 / 0.268 ms, 6.9:
        // 0.508 / 0.517 ms, 13.8: 0.993 / 1.007 ms; F64 7x7 at 3.3: 80 / 75.5 us. The walk starts at 6 tiles per slot.
        static const int persist_min_x10 = [] { const char* e = getenv("NK_TILED_PERSIST_MIN_X10"); return e ? atoi(e) : 60; }();
        // (a call that forces the TMA family -- the testing / measurement knob -- walks wherever the walk applies)
        if (p.persist && ctx->conv_path != NK_CONV_TMA && wsets == 1 && !p.wloop && tiles * 10 < slots * persist_min_x10) p.persist = 0;
        // persistent: one map per rows-per-warp value 2, 4, (8) (box of 8 r + KH - 1 rows); otherwise only the full tile's map
        for (int r = p.persist ? 2 : RH; r <= RH; r *= 2) {
            int st = nk_tma_encode(ctx, sizeof(T) == 4 ? NK_F32 : NK_F64, *img, C::SW, 8 * r + KH - 1, p.has_y != 0, &tmaps.m[nk_tmap_slot(r)]);
            if (st == -1) return -1;
            if (st) return st;
        }
        p.status = ctx->tma_status_dev;
        if (p.persist) {
            // One resident wave of CTAs: whole waves of tiles first, then the rest in 16-row units, at least one per CTA
            // (each chunk re-reads KH - 1 halo rows and pays a fixed set-up).
            ring = p.NQ < 8 && !p.wloop;   // short chunks: decoding would cost as much as the chunk's arithmetic
            if constexpr (TMA) {
                if (ring || p.wloop) {
                    // these walks run another variant of the kernel: the resident wave is what THAT variant's registers allow
                    auto kern = ring ? nk_conv_tiled_kernel<T, KH, KW, RH, true, NK_TILED_RING> : nk_conv_tiled_kernel<T, KH, KW, RH, true, NK_TILED_WLOOP>;
                    int per_sm = 1;
                    const int ost = nk_tiled_occupancy(ctx, reinterpret_cast<const void*>(kern), 288, smem, &per_sm);
                    if (ost) return ost;
                    slots = int64_t(ctx->prop.multiProcessorCount) * per_sm;
                }
            }
            grid = slots;
            if (tiles < grid) {
                grid = tiles * RH / 2;
                if (grid > slots) grid = slots;
                if (grid < 1) grid = 1;
            }
            p.waves = int(tiles / grid);
            if (tiles / grid > 0x3fffffff) return -1;
            // The tiles left after the whole waves: dealt in 16-row units while that is cheaper than one more step of whole
            // tiles for some CTAs. A short chunk runs at about half the rate of a whole tile -- with 2 rows per warp a thread
            // loads 6 row segments from shared memory per 200 multiply-adds instead of 12 per 800, which makes the chunk
            // shared-memory bound -- while the CTAs of a last whole-tile step run alone on their SMs, faster than in pairs.
            // Measured on B200 (F32 5x5, 32 channels): units win at 0.46 tiles left per CTA (3.7 %), lose from 0.8 on.
            static const int tail_pct = [] { const char* e = getenv("NK_TILED_TAIL_PCT"); return e ? atoi(e) : 50; }();
            const int64_t left = tiles - int64_t(p.waves) * grid;
            p.tail = (p.waves == 0 || left * 100 <= grid * tail_pct) ? 1 : 0;
        }
    }
    if (grid > 0x7fffffffLL) return -1;
    const unsigned threads = TMA ? 288 : 256;
    if (splits > 1 && splits <= 8) {
        // one launch: the parts of a tile as a thread-block cluster that adds itself up through shared memory
        cudaLaunchConfig_t cfg;
        memset(&cfg, 0, sizeof(cfg));
        cfg.gridDim = dim3(unsigned(grid));
        cfg.blockDim = dim3(threads);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = unsigned(splits);
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int active = 0;
        if (cudaOccupancyMaxActiveClusters(&active, nk_conv_tiled_kernel<T, KH, KW, RH, TMA>, &cfg) == cudaSuccess && active >= 1) {
            p.cluster = 1;
            T* none = nullptr;
            cudaError_t e = cudaLaunchKernelEx(&cfg, nk_conv_tiled_kernel<T, KH, KW, RH, TMA>, out, none, I, K, p, tmaps);
            if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaLaunchKernelEx(nk_conv_tiled_kernel, cluster)");
            return nk_after_launch(ctx, TMA ? "nk_conv_tiled_kernel<tma,cluster>" : "nk_conv_tiled_kernel<ldgsts,cluster>");
        }
        cudaGetLastError();   // clusters of this size do not fit: two passes instead
    }
    T* partial = nullptr;
    if (splits > 1) {
        void* scratch = nullptr;
        const size_t need = size_t(splits) * size_t(p.NP) * p.OH * p.OW * sizeof(T);
        int st = nk_scratch(ctx, need, &scratch);
        if (st) return st;
        partial = reinterpret_cast<T*>(scratch);
    }
    if constexpr (TMA) {
        if (ring) {
            nk_conv_tiled_kernel<T, KH, KW, RH, true, NK_TILED_RING><<<unsigned(grid), threads, smem, ctx->stream>>>(out, partial, I, K, p, tmaps);
            return nk_after_launch(ctx, "nk_conv_tiled_kernel<tma,ring>");
        }
        if (p.wloop) {
            nk_conv_tiled_kernel<T, KH, KW, RH, true, NK_TILED_WLOOP><<<unsigned(grid), threads, smem, ctx->stream>>>(out, partial, I, K, p, tmaps);
            return nk_after_launch(ctx, "nk_conv_tiled_kernel<tma,wloop>");
        }
    }
    nk_conv_tiled_kernel<T, KH, KW, RH, TMA><<<unsigned(grid), threads, smem, ctx->stream>>>(out, partial, I, K, p, tmaps);
    int st = nk_after_launch(ctx, TMA ? (p.persist ? "nk_conv_tiled_kernel<tma,balanced>" : "nk_conv_tiled_kernel<tma>") : "nk_conv_tiled_kernel<ldgsts>");
    if (st || splits == 1) return st;
    const int64_t plane = p.NP * int64_t(p.OH) * p.OW;
    int g = nk_grid_for(ctx, plane, 256, 8);
    nk_conv_tiled_finish_kernel<T><<<g, 256, 0, ctx->stream>>>(out, partial, p);
    return nk_after_launch(ctx, "nk_conv_tiled_finish_kernel");
}
