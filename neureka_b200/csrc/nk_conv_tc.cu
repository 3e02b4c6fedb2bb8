// Tensor-core family for F32 contraction-shaped convolution calls ([M,K,1] x [1,K,N], `Tensor.convDot`, `@`, and the two
// gradients of such calls): O[m, n] = sum_k A[m, k] * B[k, n] on the 5th-generation tensor cores with the 3xTF32 split.
// Replaces what the reference runs for these shapes on a GPU, `fast_CM_MM_MxKxN`
// (src/main/java/neureka/backend/main/operations/linear/internal/opencl/CLGEMM.java:44-92); the semantics are those of
// AbstractCPUConvolution.java:245-316 (forward) / :319-408 (deconvolution) restricted to contraction-shaped calls.
//
// 3xTF32. A TF32 operand keeps 11 significant bits, an F32 value 24. Every operand element v is split once into
// hi = tf32(v) (round to nearest) and lo = tf32(v - hi) (v - hi is exact in F32), and the product sum is evaluated as
// sum(lo_a*hi_b) + sum(hi_a*lo_b) + sum(hi_a*hi_b) with F32 accumulation in tensor memory: the dropped lo*lo term and
// the rounding of lo are below 2^-21 of |a||b| per term, inside the 1e-5 * sum|a||b| tolerance of the path.
//
// Launch sequence (one stream, one scratch block):
//   1. nk_gemm_offsets_kernel  -- the three index groups of the views flattened into offset tables (any permuted or
//      sliced view works, the drain included);
//   2. nk_tc_split_kernel x 2  -- gathers each operand through its tables into dense K-major arrays hi[rows][Kp] and
//      lo[rows][Kp] (Kp = K rounded up to 16, zero padded); the second operand is transposed on the way when its rows
//      are the contiguous direction, so both operands reach the tensor cores K-major;
//   3. nk_conv_tc_kernel       -- persistent, warp-specialised: one producer thread issues cp.async.bulk.tensor (TMA,
//      64-byte swizzle, no multicast, this GPU's memory only) into a 4-stage ring of {A_hi, A_lo, B_hi, B_lo} panels
//      of 16 k each; one thread issues tcgen05.mma (kind::tf32, M = 128, N = 256, K = 8; six per stage) into one of
//      two 128 x 256 F32 accumulators in tensor memory and hands stages back with tcgen05.commit; sixteen warps read
//      finished accumulators with tcgen05.ld and scatter the tile through the drain's tables.
//
// Accumulation. The tensor core adds each product block into the accumulator with truncation (measured: a sum of K
// same-signed terms came out low by K/8 * 3 * 2^-25 relative, 9e-5 at K = 8192). A tile's sum over k is therefore cut
// into chunks of 128 k (48 accumulations, bias below 1.5e-6): the two accumulators alternate chunk by chunk, and the
// sixteen epilogue warps add every finished chunk into per-thread F32 running sums with ordinary round-to-nearest adds
// while the next chunk's products already run into the other accumulator. The running sums of a tile (64 per thread)
// go to the drain after its last chunk.
// Every mbarrier wait is bounded (nk_mbar_wait_bounded); on expiry the waiter raises the CTA's abort word and the
// host-visible status, all roles leave their loops, outstanding copies and tensor-core work are waited for (bounded),
// tensor memory is released and the kernel returns; the host then reports NK_ERR_TIMEOUT.
#include <cuda.h>

#include "nk_gemm_plan.h"
#include "nk_ptx.cuh"

int nk_tma_encode_2d_f32(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, int box_cols, int box_rows, int swizzle,
                         CUtensorMap* out);

namespace {

constexpr int TC_BM = 128, TC_BN = 256, TC_BK = 16, TC_STAGES = 4;
constexpr int TC_A_PART = TC_BM * TC_BK * 4;                 // 8 KiB: one of A_hi / A_lo for a stage
constexpr int TC_B_PART = TC_BN * TC_BK * 4;                 // 16 KiB
constexpr int TC_STAGE_BYTES = 2 * TC_A_PART + 2 * TC_B_PART;   // 48 KiB
constexpr int TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int TC_THREADS = 576;                              // warp 0 producer, warp 1 tensor-core issue, warps 2..17 epilogue
constexpr int TC_EPI_COLS = 64;                              // accumulator columns an epilogue warp owns (4 warps per lane quarter)
constexpr unsigned TC_TMEM_COLS = 512;                       // two 128 x 256 F32 accumulators
constexpr int TC_KC = 8;                                     // k blocks (of 16) per accumulation chunk

// ---- split: v -> hi = tf32(v), lo = tf32(v - hi) ------------------------------------------------------------------------
__device__ __forceinline__ void tc_split(float v, float* hi, float* lo) {
    unsigned h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(v));
    float fh = __uint_as_float(h);
    if (!isfinite(fh)) fh = isfinite(v) ? __uint_as_float(__float_as_uint(v) & 0xffffe000u) : v;   // rounded past the largest finite value
    float r = isfinite(v) ? v - fh : 0.0f;
    unsigned l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(r));
    *hi = fh;
    *lo = __uint_as_float(l);
}

// Gathers src[base + offR[r] + offK[k]] into hi / lo [R][Kp], zero for k >= K. KFAST: consecutive k are consecutive
// in memory (threads run along k); otherwise threads run along the rows on the way in and the 32 x 32 tile is
// transposed through shared memory, so both the reads and the writes stay coalesced.
template <bool KFAST>
__global__ void __launch_bounds__(256) nk_tc_split_kernel(const float* __restrict__ src, int64_t base, const int64_t* __restrict__ offR,
                                                          const int64_t* __restrict__ offK, int64_t R, int64_t K, int64_t Kp,
                                                          float* __restrict__ hi, float* __restrict__ lo) {
    __shared__ float tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t r0 = int64_t(blockIdx.x) * 32, k0 = int64_t(blockIdx.y) * 32;
    if (KFAST) {
        const int64_t k = k0 + tx;
        const int64_t ok = k < K ? offK[k] : 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t r = r0 + ty + 8 * i;
            if (r >= R || k >= Kp) continue;
            const float v = k < K ? src[base + offR[r] + ok] : 0.0f;
            float h, l;
            tc_split(v, &h, &l);
            hi[r * Kp + k] = h;
            lo[r * Kp + k] = l;
        }
    } else {
        const int64_t rr = r0 + tx;
        const int64_t orr = rr < R ? offR[rr] : 0;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t k = k0 + ty + 8 * i;
            tile[ty + 8 * i][tx] = (rr < R && k < K) ? src[base + orr + offK[k]] : 0.0f;
        }
        __syncthreads();
        const int64_t k = k0 + tx;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int64_t r = r0 + ty + 8 * i;
            if (r >= R || k >= Kp) continue;
            float h, l;
            tc_split(tile[tx][ty + 8 * i], &h, &l);
            hi[r * Kp + k] = h;
            lo[r * Kp + k] = l;
        }
    }
}

// ---- tcgen05 wrappers ------------------------------------------------------------------------------------------------
// Shared-memory operand descriptor, K-major, 64-byte swizzle: rows of 64 bytes (16 F32), 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t tc_smem_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= uint64_t((saddr & 0x3ffffu) >> 4);     // start address, 16-byte units
    d |= uint64_t(1) << 16;                     // leading byte offset: not used by swizzled K-major layouts
    d |= uint64_t(512 >> 4) << 32;              // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                     // descriptor version of this architecture
    d |= uint64_t(4) << 61;                     // layout type: 64-byte swizzle
    return d;
}
// Instruction descriptor: F32 accumulate, TF32 x TF32, both operands K-major, N = 256, M = 128.
constexpr uint32_t TC_IDESC = (1u << 4) | (2u << 7) | (2u << 10) | (uint32_t(TC_BN >> 3) << 17) | (uint32_t(TC_BM >> 4) << 24);

__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(da), "l"(db), "r"(TC_IDESC), "r"(accumulate) : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    unsigned a = (unsigned)__cvta_generic_to_shared(bar);
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(a) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// 16 consecutive accumulator columns of this thread's lane (32 lanes x 32 bits per warp and column)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
                   "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

struct TcParams {
    int64_t M, N;
    int k_blocks;                  // Kp / 16
    int tiles_m;
    int64_t tiles;
    const int64_t* offOm;
    const int64_t* offOn;
    int64_t bO;
    int out_vec;                   // the drain's n index is its contiguous direction and every row starts 16-byte aligned
    int* status;                   // host-mapped word, set non-zero when a bounded wait ran out
};

__global__ void __launch_bounds__(TC_THREADS, 1)
nk_conv_tc_kernel(float* __restrict__ out, const __grid_constant__ CUtensorMap mAhi, const __grid_constant__ CUtensorMap mAlo,
                  const __grid_constant__ CUtensorMap mBhi, const __grid_constant__ CUtensorMap mBlo, const TcParams p) {
    extern __shared__ unsigned char tc_smem_raw[];
    // stages must start on a 1024-byte boundary (swizzle pattern = function of the address bits)
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TC_STAGES * TC_STAGE_BYTES);
    uint64_t* full_bar = bars;                         // [STAGES] a stage's four panels have landed
    uint64_t* empty_bar = bars + TC_STAGES;            // [STAGES] the products reading a stage have completed
    uint64_t* acc_full = bars + 2 * TC_STAGES;         // [2] an accumulator holds a finished tile
    uint64_t* acc_empty = bars + 2 * TC_STAGES + 2;    // [2] the epilogue has read it out
    uint64_t* drain_bar = bars + 2 * TC_STAGES + 4;    // only on the abort path: all issued products have completed
    volatile int* abort_word = reinterpret_cast<volatile int*>(bars + 2 * TC_STAGES + 5);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * TC_STAGES + 6);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < TC_STAGES; s++) { nk_mbar_init(&full_bar[s], 1); nk_mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; b++) { nk_mbar_init(&acc_full[b], 1); nk_mbar_init(&acc_empty[b], 16); }
        nk_mbar_init(drain_bar, 1);
        *abort_word = 0;
        nk_fence_barrier_init();
        nk_fence_proxy_async();
    }
    if (warp == 1) {   // one warp allocates all of the SM's tensor memory (one CTA per SM: 192 KiB of shared memory each)
        unsigned slot = (unsigned)__cvta_generic_to_shared(tmem_slot);
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(slot), "r"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    auto wait_or_abort = [&](uint64_t* bar, unsigned parity) -> bool {
        const int r = nk_mbar_wait_bounded(bar, parity, NK_WAIT_LIMIT_NS, abort_word);
        if (r < 0) {
            *abort_word = 1;
            if (p.status) atomicExch(p.status, 1);
        }
        return r > 0;
    };

    if (warp == 0) {
        if (lane == 0) {
            // ---- producer: four tensor copies per stage ----
            int it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {
                const int m0 = int(t % p.tiles_m) * TC_BM, n0 = int(t / p.tiles_m) * TC_BN;
                for (int kb = 0; kb < p.k_blocks && ok; kb++, it++) {
                    const int s = it % TC_STAGES;
                    ok = wait_or_abort(&empty_bar[s], ((unsigned(it) / TC_STAGES) & 1u) ^ 1u);
                    if (!ok) break;
                    unsigned char* st = smem + size_t(s) * TC_STAGE_BYTES;
                    nk_mbar_expect_tx(&full_bar[s], unsigned(TC_STAGE_BYTES));
                    const int k0 = kb * TC_BK;
                    nk_tma_load_2d(st, &mAhi, &full_bar[s], k0, m0);
                    nk_tma_load_2d(st + TC_A_PART, &mAlo, &full_bar[s], k0, m0);
                    nk_tma_load_2d(st + 2 * TC_A_PART, &mBhi, &full_bar[s], k0, n0);
                    nk_tma_load_2d(st + 2 * TC_A_PART + TC_B_PART, &mBlo, &full_bar[s], k0, n0);
                }
            }
            if (!ok || *abort_word) {
                // copies already requested still land in this CTA's shared memory: wait for them (bounded)
                for (int j = (it > TC_STAGES ? it - TC_STAGES : 0); j < it; j++)
                    nk_mbar_wait_bounded(&full_bar[j % TC_STAGES], (unsigned(j) / TC_STAGES) & 1u, NK_WAIT_LIMIT_NS, nullptr);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // ---- tensor-core issue: per stage two k-steps of 8, three products each (small terms first); a new
            // accumulator every TC_KC stages ----
            int it = 0, ch = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {
                for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += TC_KC, ch++) {
                    const int b = ch & 1;
                    ok = wait_or_abort(&acc_empty[b], ((unsigned(ch) >> 1) & 1u) ^ 1u);
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t acc = tmem_base + uint32_t(b) * TC_BN;
                    const int kb1 = kb0 + TC_KC < p.k_blocks ? kb0 + TC_KC : p.k_blocks;
                    for (int kb = kb0; kb < kb1 && ok; kb++, it++) {
                        const int s = it % TC_STAGES;
                        ok = wait_or_abort(&full_bar[s], (unsigned(it) / TC_STAGES) & 1u);
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem + size_t(s) * TC_STAGE_BYTES);
#pragma unroll
                        for (int ks = 0; ks < TC_BK / 8; ks++) {
                            const uint32_t koff = uint32_t(ks) * 32u;   // 8 F32 further along the 64-byte row
                            const uint64_t a_hi = tc_smem_desc(sa + koff), a_lo = tc_smem_desc(sa + TC_A_PART + koff);
                            const uint64_t b_hi = tc_smem_desc(sa + 2 * TC_A_PART + koff), b_lo = tc_smem_desc(sa + 2 * TC_A_PART + TC_B_PART + koff);
                            tc_mma(acc, a_lo, b_hi, (kb > kb0 || ks != 0) ? 1u : 0u);
                            tc_mma(acc, a_hi, b_lo, 1u);
                            tc_mma(acc, a_hi, b_hi, 1u);
                        }
                        tc_commit(&empty_bar[s]);       // the stage goes back to the producer when these products are done
                    }
                    if (ok) tc_commit(&acc_full[b]);    // ... and the chunk to the epilogue
                }
            }
            if (!ok || *abort_word) {
                tc_commit(drain_bar);               // nothing of this CTA may still run on the tensor cores at release time
                nk_mbar_wait_bounded(drain_bar, 0, NK_WAIT_LIMIT_NS, nullptr);
            }
        }
    } else {
        // ---- epilogue: warps 2..17; warp w reads the 32 accumulator lanes of its quarter (w % 4) and the 64 columns of
        // part (w - 2) / 4, adds every finished chunk into its running sums and stores them after the tile's last chunk ----
        const int q = warp & 3, half = (warp - 2) >> 2;
        int ch = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < p.tiles && ok; t += gridDim.x) {
            const int64_t m = int64_t(t % p.tiles_m) * TC_BM + q * 32 + lane;
            const int64_t n0 = int64_t(t / p.tiles_m) * TC_BN + half * TC_EPI_COLS;
            float sum[TC_EPI_COLS];
            for (int kb0 = 0; kb0 < p.k_blocks && ok; kb0 += TC_KC, ch++) {
                const int b = ch & 1;
                ok = wait_or_abort(&acc_full[b], (unsigned(ch) >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                const uint32_t src = tmem_base + (uint32_t(q * 32) << 16) + uint32_t(b) * TC_BN + uint32_t(half) * TC_EPI_COLS;
#pragma unroll
                for (int c = 0; c < TC_EPI_COLS / 16; c++) {
                    uint32_t v[16];
                    tc_ld16(src + uint32_t(c) * 16u, v);
                    if (kb0 == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j++) sum[c * 16 + j] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j++) sum[c * 16 + j] += __uint_as_float(v[j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) nk_mbar_arrive(&acc_empty[b]);
            }
            if (!ok || m >= p.M) continue;
            const int64_t row = p.bO + p.offOm[m];
#pragma unroll
            for (int c = 0; c < TC_EPI_COLS / 32; c++) {
                const int64_t n = n0 + c * 32;
                if (n >= p.N) continue;
                if (p.out_vec && n + 32 <= p.N) {
                    float4* dst = reinterpret_cast<float4*>(out + row + n);
#pragma unroll
                    for (int j = 0; j < 8; j++) dst[j] = make_float4(sum[c * 32 + 4 * j], sum[c * 32 + 4 * j + 1], sum[c * 32 + 4 * j + 2], sum[c * 32 + 4 * j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++)
                        if (n + j < p.N) out[row + p.offOn[n + j]] = sum[c * 32 + j];
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
    }
}

}  // namespace

int nk_conv_tc_try(nk_ctx* ctx, nk_buf* drn, nk_buf* s1, nk_buf* s2, const GemmPlan& p, bool* handled) {
    *handled = false;
    const bool forced = ctx->conv_path == NK_CONV_TC;
    // worth three extra launches and a pass over both operands only for real matrix products
    if (p.M < 64 || p.N < 64 || p.K < 32) return NK_OK;
    if (!forced && double(p.M) * double(p.N) * double(p.K) < double(1 << 24)) return NK_OK;
    if (p.K >= (int64_t(1) << 21) || p.M >= (int64_t(1) << 31) || p.N >= (int64_t(1) << 31)) return NK_OK;
    const int64_t Kp = ((p.K + TC_BK - 1) / TC_BK) * TC_BK;
    const int64_t tiles_m = (p.M + TC_BM - 1) / TC_BM, tiles_n = (p.N + TC_BN - 1) / TC_BN;
    if (tiles_m * tiles_n > 0x7fffffffLL) return NK_OK;
    if (size_t(TC_SMEM_BYTES) > size_t(ctx->prop.sharedMemPerBlockOptin)) return NK_OK;

    // scratch: [tables | A_hi | A_lo | B_hi | B_lo], the arrays on 1024-byte boundaries
    const size_t tab_bytes = ((size_t(2 * (p.M + p.N + p.K)) * sizeof(int64_t) + 1023) / 1024) * 1024;
    const size_t a_bytes = ((size_t(p.M) * Kp * 4 + 1023) / 1024) * 1024, b_bytes = ((size_t(p.N) * Kp * 4 + 1023) / 1024) * 1024;
    void* scratch = nullptr;
    int st = nk_scratch(ctx, tab_bytes + 2 * a_bytes + 2 * b_bytes + 1024, &scratch);
    if (st) return st;
    scratch = reinterpret_cast<void*>((reinterpret_cast<uintptr_t>(scratch) + 1023) & ~uintptr_t(1023));
    int64_t* tab = reinterpret_cast<int64_t*>(scratch);
    char* base = reinterpret_cast<char*>(scratch) + tab_bytes;
    float *Ahi = reinterpret_cast<float*>(base), *Alo = reinterpret_cast<float*>(base + a_bytes);
    float *Bhi = reinterpret_cast<float*>(base + 2 * a_bytes), *Blo = reinterpret_cast<float*>(base + 2 * a_bytes + b_bytes);

    CUtensorMap mAhi, mAlo, mBhi, mBlo;
    if (nk_tma_encode_2d_f32(Ahi, uint64_t(p.M), uint64_t(Kp), uint64_t(Kp) * 4, TC_BK, TC_BM, 2, &mAhi) ||
        nk_tma_encode_2d_f32(Alo, uint64_t(p.M), uint64_t(Kp), uint64_t(Kp) * 4, TC_BK, TC_BM, 2, &mAlo) ||
        nk_tma_encode_2d_f32(Bhi, uint64_t(p.N), uint64_t(Kp), uint64_t(Kp) * 4, TC_BK, TC_BN, 2, &mBhi) ||
        nk_tma_encode_2d_f32(Blo, uint64_t(p.N), uint64_t(Kp), uint64_t(Kp) * 4, TC_BK, TC_BN, 2, &mBlo))
        return NK_OK;   // no tensor-map encoder: the FMA family takes the call

    st = nk_gemm_build_tables(ctx, p, tab);
    if (st) return st;
    const int64_t *offA_m = tab, *offO_m = tab + p.M, *offB_n = tab + 2 * p.M, *offO_n = tab + 2 * p.M + p.N;
    const int64_t *offA_k = tab + 2 * p.M + 2 * p.N, *offB_k = tab + 2 * p.M + 2 * p.N + p.K;

    // is k the contiguous direction of an operand? (the innermost dim of its k group has stride 1)
    const bool a_kfast = p.k.n > 0 && p.k.sa[p.k.n - 1] == 1;
    const bool b_kfast = p.k.n > 0 && p.k.sb[p.k.n - 1] == 1;
    const dim3 ga(unsigned((p.M + 31) / 32), unsigned((Kp + 31) / 32)), gb(unsigned((p.N + 31) / 32), unsigned((Kp + 31) / 32));
    const float* A = static_cast<const float*>(s1->ptr);
    const float* B = static_cast<const float*>(s2->ptr);
    if (a_kfast) nk_tc_split_kernel<true><<<ga, 256, 0, ctx->stream>>>(A, p.bA, offA_m, offA_k, p.M, p.K, Kp, Ahi, Alo);
    else nk_tc_split_kernel<false><<<ga, 256, 0, ctx->stream>>>(A, p.bA, offA_m, offA_k, p.M, p.K, Kp, Ahi, Alo);
    if ((st = nk_after_launch(ctx, "nk_tc_split_kernel"))) return st;
    if (b_kfast) nk_tc_split_kernel<true><<<gb, 256, 0, ctx->stream>>>(B, p.bB, offB_n, offB_k, p.N, p.K, Kp, Bhi, Blo);
    else nk_tc_split_kernel<false><<<gb, 256, 0, ctx->stream>>>(B, p.bB, offB_n, offB_k, p.N, p.K, Kp, Bhi, Blo);
    if ((st = nk_after_launch(ctx, "nk_tc_split_kernel"))) return st;

    TcParams tp;
    tp.M = p.M; tp.N = p.N;
    tp.k_blocks = int(Kp / TC_BK);
    tp.tiles_m = int(tiles_m);
    tp.tiles = tiles_m * tiles_n;
    tp.offOm = offO_m; tp.offOn = offO_n;
    tp.bO = p.bO;
    bool vec = p.n.n == 1 && p.n.sb[0] == 1 && (p.bO % 4) == 0 && (reinterpret_cast<uintptr_t>(drn->ptr) % 16) == 0;
    for (int d = 0; d < p.m.n && vec; d++) vec = (p.m.sb[d] % 4) == 0;
    tp.out_vec = vec ? 1 : 0;
    tp.status = ctx->tma_status_dev;

    cudaError_t e = cudaFuncSetAttribute(nk_conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM_BYTES);
    if (e != cudaSuccess) return nk_cuda_fail(ctx, e, "cudaFuncSetAttribute(nk_conv_tc_kernel)");
    const int64_t sms = ctx->prop.multiProcessorCount;
    const unsigned grid = unsigned(tp.tiles < sms ? tp.tiles : sms);
    nk_conv_tc_kernel<<<grid, TC_THREADS, TC_SMEM_BYTES, ctx->stream>>>(static_cast<float*>(drn->ptr), mAhi, mAlo, mBhi, mBlo, tp);
    if ((st = nk_after_launch(ctx, "nk_conv_tc_kernel<3xtf32>"))) return st;
    *handled = true;
    return NK_OK;
}
