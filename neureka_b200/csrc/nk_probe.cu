// Measured arithmetic ceilings of the device the context runs on: a register-resident FMA loop with enough
// independent chains to saturate the pipe. The benchmark uses the results as roofline denominators for the
// FP32-FMA-bound stencil and the FP64-bound kernels (F64 convolution, the double-evaluated activations).
#include "nk_internal.h"
#include "nk_conv_tiled.cuh"

template <class T>
__global__ void __launch_bounds__(256) nk_fma_peak_kernel(T* __restrict__ sink, int iters, T seed) {
    T a[16];
#pragma unroll
    for (int k = 0; k < 16; k++) a[k] = seed + T(threadIdx.x + k);
    const T m = T(0.999999), c = T(1e-7);
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 16; k++) a[k] = fma(a[k], m, c);
    }
    T s = 0;
#pragma unroll
    for (int k = 0; k < 16; k++) s += a[k];
    if (s == T(-1)) sink[0] = s;   // never true: keeps the loop alive without a store
}

extern "C" int nk_measure_fma_peak(nk_ctx* ctx, int32_t dtype, double* out_tflops) {
    NK_CHECK_CTX(ctx);
    if (!out_tflops) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_measure_fma_peak: out pointer is null");
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(ctx, NK_ERR_UNSUPPORTED, "nk_measure_fma_peak: F32/F64 only");
    void* sink = nullptr;
    int st = nk_scratch(ctx, 64, &sink);
    if (st) return st;
    const int grid = ctx->prop.multiProcessorCount * 8, block = 256;
    const int iters = dtype == NK_F32 ? 8192 : 2048;
    float best = 1e30f;
    for (int rep = 0; rep < 4; rep++) {
        NK_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
        if (dtype == NK_F32) nk_fma_peak_kernel<float><<<grid, block, 0, ctx->stream>>>((float*)sink, iters, 1.0f);
        else nk_fma_peak_kernel<double><<<grid, block, 0, ctx->stream>>>((double*)sink, iters, 1.0);
        st = nk_after_launch(ctx, "nk_fma_peak_kernel");
        if (st) return st;
        NK_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
        NK_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
        float ms = 0;
        NK_CUDA(ctx, cudaEventElapsedTime(&ms, ctx->ev0, ctx->ev1));
        if (rep > 0 && ms < best) best = ms;
    }
    const double flops = 2.0 * 16.0 * double(iters) * double(grid) * block;
    *out_tflops = flops / (double(best) * 1e-3) / 1e12;
    return NK_OK;
}


// ---- the bounded wait the pipelined kernels rely on, exercised on its own ------------------------------------------
// One warp initialises an mbarrier that nothing will ever arrive on and waits for it with the same helper and the same
// reporting path (abort word, host-mapped status word) as the convolution kernels, with a limit given by the caller.
// The kernel must return after about limit_ns and the next synchronising call must report NK_ERR_TIMEOUT.
__global__ void nk_wait_probe_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    if (threadIdx.x == 0) {
        nk_mbar_init(&bar, 1);
        abort_word = 0;
        nk_fence_barrier_init();
    }
    __syncthreads();
    const unsigned long long t0 = nk_globaltimer_ns();
    const int r = nk_mbar_wait_bounded(&bar, 0, limit_ns, &abort_word);
    if (r < 0) {
        abort_word = 1;
        if (status) atomicExch(status, 1);
    }
    if (threadIdx.x == 0 && waited_ns) *waited_ns = nk_globaltimer_ns() - t0;
}

extern "C" int nk_probe_wait_timeout(nk_ctx* ctx, uint64_t limit_ns, uint64_t* out_waited_ns) {
    NK_CHECK_CTX(ctx);
    if (limit_ns == 0 || limit_ns > 1000000000ull) return nk_fail(ctx, NK_ERR_BAD_ARG, "nk_probe_wait_timeout: limit must be 1 ns .. 1 s");
    void* scratch = nullptr;
    int st = nk_scratch(ctx, 64, &scratch);
    if (st) return st;
    nk_wait_probe_kernel<<<1, 32, 0, ctx->stream>>>(limit_ns, ctx->tma_status_dev, reinterpret_cast<unsigned long long*>(scratch));
    st = nk_after_launch(ctx, "nk_wait_probe_kernel");
    if (st) return st;
    NK_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (out_waited_ns) NK_CUDA(ctx, cudaMemcpy(out_waited_ns, scratch, sizeof(uint64_t), cudaMemcpyDeviceToHost));
    return NK_OK;   // the expired wait is reported by the next nk_sync / nk_read, like a kernel's would be
}
