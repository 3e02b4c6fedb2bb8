/*
 * neureka_cuda.h -- C ABI of libneureka_cuda, the CUDA (sm_100a) backend library for Neureka's
 * convolution / broadcast / elementwise path.
 *
 * This is the boundary a JVM-side `CudaDevice` / `CudaBackend` binds (Panama FFM or JNI): plain
 * pointers, sizes and int codes only. Every entry point names the reference interface it replaces;
 * paths are relative to the reference project root, J = src/main/java/neureka.
 *
 * Conventions
 *  - Every function returns an nk_status (0 = ok). A non-zero status leaves a message readable with
 *    nk_last_error(). Nothing aborts the process and no kernel traps.
 *  - A view descriptor ("cfg") is `const int32_t cfg[5*rank]`, exactly NDConfiguration.asInlineArray():
 *    [ shape | strides | indicesMap | offset | spread ]  (J/ndim/config/NDConfiguration.java:335-345).
 *    All offset arithmetic inside the library is 64-bit. Views are validated against the buffer size
 *    before any launch; an out-of-range view yields NK_ERR_BOUNDS instead of a fault.
 *  - `d` is Arg.DerivIdx exactly as the Java side holds it (J/backend/api/Call.java:107):
 *    d < 0 forward, d >= 0 derivative / deconvolution variant.
 *  - Kernels are asynchronous on the context's stream; nk_read() and nk_sync() synchronise
 *    ("stream-ordered, sync on read", like the in-order queue of J/devices/opencl/OpenCLDevice.java:140-145).
 *  - The library never computes on the CPU: without a usable CUDA device nk_device_open fails.
 */
#ifndef NEUREKA_CUDA_H
#define NEUREKA_CUDA_H

#include <stdint.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct nk_ctx nk_ctx; /* one CUDA device + one stream; replaces an OpenCLDevice's queue */
typedef struct nk_buf nk_buf; /* one device allocation; replaces a cl_mem held by OpenCLDevice.cl_tsr */

typedef enum {
    NK_OK = 0,
    NK_ERR_BAD_ARG = 1,     /* -> IllegalArgumentException */
    NK_ERR_UNSUPPORTED = 2, /* dtype / rank / op not supported -> IllegalArgumentException */
    NK_ERR_OOM = 3,         /* cudaErrorMemoryAllocation -> OutOfMemoryError-like */
    NK_ERR_CUDA = 4,        /* any other CUDA failure -> IllegalStateException */
    NK_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out */
    NK_ERR_BOUNDS = 6       /* a view reaches outside its buffer -> IllegalArgumentException */
} nk_status;

typedef enum { NK_F32 = 0, NK_F64 = 1, NK_I8 = 2, NK_I16 = 3, NK_I32 = 4, NK_I64 = 5 } nk_dtype;

/* Binary operators: Addition, Subtraction, Multiplication, Division, Modulo, Power
 * (J/backend/main/operations/operator/*.java), IDY = AssignLeft's scalar form
 * (J/backend/main/implementations/broadcast/CPUScalarBroadcastIdentity.java). */
typedef enum { NK_OP_ADD = 0, NK_OP_SUB = 1, NK_OP_MUL = 2, NK_OP_DIV = 3, NK_OP_MOD = 4, NK_OP_POW = 5, NK_OP_IDY = 6,
               /* handle*drain product for both derivative slots: the TestBroadcast implementation of
                  src/test/java/testutility/UnitTester_Tensor.java:414-433; only valid for nk_broadcast */
               NK_OP_MUL_BOTH = 7 } nk_op;

/* The 23 ScalarFun ids (J/backend/main/implementations/fun/api/ScalarFun.java:5-29), alphabetical by id(). */
typedef enum {
    NK_FUN_ABS = 0, NK_FUN_CBRT, NK_FUN_COS, NK_FUN_EXP, NK_FUN_GASU, NK_FUN_GATU, NK_FUN_GAUS, NK_FUN_FAST_GAUS,
    NK_FUN_GELU, NK_FUN_IDY, NK_FUN_LOG10, NK_FUN_LN, NK_FUN_QUAD, NK_FUN_RELU, NK_FUN_SELU, NK_FUN_SILU, NK_FUN_SIG,
    NK_FUN_SIN, NK_FUN_SOFTPLUS, NK_FUN_SOFTSIGN, NK_FUN_SQRT, NK_FUN_TANH, NK_FUN_FAST_TANH, NK_FUN_COUNT
} nk_fun;

/* Which convolution kernel family a call is routed to. AUTO picks from the views; the others force a
 * family (NK_ERR_UNSUPPORTED if the views do not qualify) -- a testing/measurement knob. Forcing NK_CONV_TMA also
 * selects the persistent tile walk wherever it applies (AUTO keeps one tile per CTA below 6 tiles per resident CTA). */
typedef enum { NK_CONV_AUTO = 0, NK_CONV_GENERIC = 1, NK_CONV_TILED = 2, NK_CONV_TMA = 3, NK_CONV_GEMM = 4, NK_CONV_TC = 5 } nk_conv_path;

typedef struct {
    char name[256];
    uint64_t total_mem_bytes;
    int32_t sm_count;
    int32_t cc_major, cc_minor;
    int32_t l2_bytes;
    int32_t max_smem_per_block;
    int32_t clock_khz;
} nk_props;

/* ---- lifecycle: replaces OpenCLPlatform/OpenCLDevice discovery + queue creation
 *      (J/devices/opencl/OpenCLPlatform.java:60-110, J/devices/opencl/OpenCLDevice.java:140-160) ---- */
int nk_device_count(int32_t* out_count);
int nk_device_open(int32_t ordinal, nk_ctx** out_ctx);
int nk_device_close(nk_ctx* ctx);                 /* Device.dispose(), J/devices/Device.java:155 */
int nk_device_props(nk_ctx* ctx, nk_props* out);  /* OpenCLDevice.name()/globalMemSize()..., OpenCLDevice.java:728-900 */
int nk_sync(nk_ctx* ctx);                         /* clFinish equivalent */
void* nk_stream(nk_ctx* ctx);                     /* the cudaStream_t launches go to (for interop) */
/* Message of the last failure on ctx (or of the calling thread when ctx is NULL). Never NULL. */
const char* nk_last_error(nk_ctx* ctx);
const char* nk_version(void);

/* ---- memory: replaces OpenCLDevice._add/_store/free/access
 *      (OpenCLDevice.java:355-405 store, :497-524 free, :553-594 allocate*, :616-632 overwrite,
 *       :676-690 read; Device.Access J/devices/Device.java:305-407) ---- */
/* Device.allocate(DataType, size). Blocks come from the device's stream-ordered memory pool and go back to it on
 * nk_free, in the order of ctx's stream: neither call waits for the device, and a freed block is handed out again
 * without a trip to the driver (the reference creates and releases one cl_mem per tensor, OpenCLDevice.java:385-405,
 * :497-524). A buffer used by a second context's stream must be ordered against ctx's stream with nk_event_*. */
int nk_alloc(nk_ctx* ctx, int32_t dtype, int64_t n_elems, nk_buf** out);
/* The same from the driver's plain allocator: the only kind of buffer nk_ipc_export accepts. nk_free of such a buffer
 * waits for the device. (No reference counterpart.) */
int nk_alloc_shared(nk_ctx* ctx, int32_t dtype, int64_t n_elems, nk_buf** out);
int nk_wrap(nk_ctx* ctx, int32_t dtype, void* device_ptr, int64_t n_elems, nk_buf** out); /* adopt foreign device memory, not owned */
int nk_free(nk_ctx* ctx, nk_buf* buf);                                       /* Device.free; NULL is a no-op */
int nk_buf_info(nk_buf* buf, void** device_ptr, int64_t* n_elems, int32_t* dtype);
/* Access.write(item).intoRange(start, start+n): fill n elements with one value (allocateFromOne) */
int nk_fill(nk_ctx* ctx, nk_buf* buf, double value, int64_t start, int64_t n);
/* Access.writeFrom(array, host_off).intoRange(dev_start, dev_start+n); blocking w.r.t. the host array */
int nk_write(nk_ctx* ctx, nk_buf* buf, const void* host, int64_t host_off, int64_t dev_start, int64_t n);
/* Access.readArray(type, dev_start, n) / readAll; blocking */
int nk_read(nk_ctx* ctx, nk_buf* buf, void* host, int64_t dev_start, int64_t n);
/* device-to-device range copy on the stream (used by swap/actualize; OpenCLDevice.java:574-594) */
int nk_copy(nk_ctx* ctx, nk_buf* dst, int64_t dst_start, nk_buf* src, int64_t src_start, int64_t n);
/* page-locked host staging memory + asynchronous variants (new: the reference's transfers are all blocking) */
int nk_host_alloc(size_t bytes, void** out_host);
int nk_host_free(void* host);
int nk_write_async(nk_ctx* ctx, nk_buf* buf, const void* pinned_host, int64_t host_off, int64_t dev_start, int64_t n);
int nk_read_async(nk_ctx* ctx, nk_buf* buf, void* pinned_host, int64_t dev_start, int64_t n);

/* ---- kernels: each replaces one CLImplementation + its .cl template ---- */

/* Operations "x", "«x", "x»" on algorithm NDConvolution: replaces CLConvolution
 * (J/backend/main/implementations/convolution/CLConvolution.java:10-32 + resources/kernels/convolution_template.cl)
 * with the semantics of the CPU implementation (AbstractCPUConvolution.java:70-143 forward, :146-240 deconvolution).
 * drn/src1/src2 = call.input(0..2) after ConvUtil's input rearrangement; all three have `rank` dims. */
int nk_conv(nk_ctx* ctx, int32_t dtype, int32_t rank,
            nk_buf* drn, const int32_t* cfg0, nk_buf* src1, const int32_t* cfg1, nk_buf* src2, const int32_t* cfg2,
            int32_t d);

/* Algorithm Broadcast: replaces CLBroadcast* (J/backend/main/implementations/broadcast/CLBroadcast.java:10-33 +
 * kernels/broadcast_template.cl), semantics of CPUBroadcast.java:62-160. d<0: drn = f(a,b) with broadcasting;
 * d>=0: (origin, handle, drain) reduction over the dims where origin is smaller. */
int nk_broadcast(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                 nk_buf* drn, const int32_t* cfg0, nk_buf* a, const int32_t* cfg1, nk_buf* b, const int32_t* cfg2,
                 int32_t d);

/* Algorithm BiElementwise: replaces CLBiElementwise* (J/backend/main/implementations/elementwise/CLBiElementwise.java:7-32 +
 * kernels/elementwise_template.cl), semantics of CPUBiElementWise.java:56-140. */
int nk_binary(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
              nk_buf* drn, const int32_t* cfg0, nk_buf* a, const int32_t* cfg1, nk_buf* b, const int32_t* cfg2,
              int32_t d);

/* Algorithm ElementwiseAlgorithm for the 23 activations and AssignLeft (fun = NK_FUN_IDY): replaces
 * CLElementwiseFunction (J/backend/main/implementations/elementwise/CLElementwiseFunction.java:12-42 +
 * kernels/activation_template.cl), semantics of CPUElementwiseFunction.java:30-116. */
int nk_unary(nk_ctx* ctx, int32_t fun, int32_t dtype, int32_t rank,
             nk_buf* drn, const int32_t* cfg0, nk_buf* src, const int32_t* cfg1, int32_t d);

/* Algorithm BiScalarBroadcast: replaces CLScalarBroadcast* (J/backend/main/implementations/broadcast/CLScalarBroadcast.java:16-64 +
 * kernels/scalarization_template.cl), semantics of CPUScalarBroadcast.java:29-75: drn = f(src, value). */
int nk_scalar_binary(nk_ctx* ctx, int32_t op, int32_t dtype, int32_t rank,
                     nk_buf* drn, const int32_t* cfg0, nk_buf* src, const int32_t* cfg1, double value, int32_t d);

/* Algorithm ScalarBroadcast: replaces the inline OpenCL wiring of J/backend/main/algorithms/ScalarBroadcast.java:65-82 +
 * kernels/scalar_broadcast.cl: every element of the drain view := fun(value) (or fun'(value) for d>=0).
 * fun(value) is evaluated on the device by one thread and broadcast. */
int nk_fill_fun(nk_ctx* ctx, int32_t fun, int32_t dtype, int32_t rank, nk_buf* drn, const int32_t* cfg0,
                double value, int32_t d);

/* Algorithm SumAlgorithm: replaces CLSum (J/backend/main/operations/linear/internal/opencl/CLSum.java:23-132):
 * out[out_index] = sum of the n elements of the view, 128-wide tiles reduced recursively in the order of
 * CPUSum (J/backend/main/operations/other/internal/CPUSum.java:26-76). */
int nk_sum(nk_ctx* ctx, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out, int64_t out_index);

/* No counterpart in the reference. The same sum as nk_sum (same tiles, same order of additions, identical result)
 * for callers that must not trigger a device allocation: hosts that have given all of the GPU's memory to their own
 * tensor pool, where nk_sum's grow-on-demand scratch block could fail or stall the device in the middle of a pass.
 * The partial sums live in a fixed array of NK_SUM_STATIC_SCRATCH_BYTES that every GPU loading the library holds
 * until exit. Limits and rules:
 *  - the view may have at most about 16.6 million F64 / 33.2 million F32 elements (ceil(n/128) + ceil(n/128^2) + 2
 *    partial sums must fit the array); larger views are rejected with NK_ERR_UNSUPPORTED -- use nk_sum for them;
 *  - the first call on a device looks up the array's device address; make that first call outside any stream capture;
 *  - all calls on a device share the array (it keeps the previous call's partial sums; nothing needs clearing, every
 *    level is rewritten before it is read), so calls that overlap on the GPU race: order them on one stream;
 *  - the call performs no cudaMalloc/cudaFree and calls no allocating library routine. */
#define NK_SUM_STATIC_SCRATCH_BYTES (1 << 20)
int nk_sum_static(nk_ctx* ctx, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out, int64_t out_index);

/* ---- routing knobs / introspection (no reference counterpart; measurement support) ---- */
int nk_set_conv_path(nk_ctx* ctx, int32_t path);        /* nk_conv_path */
int nk_last_conv_path(nk_ctx* ctx, int32_t* out_path);   /* family the last nk_conv used */
const char* nk_last_kernel(nk_ctx* ctx);                 /* name of the last kernel launched */
int nk_launch_count(nk_ctx* ctx, uint64_t* out);         /* kernels launched by this ctx so far */
int nk_timer_begin(nk_ctx* ctx);                         /* CUDA event on the ctx stream */
int nk_timer_end(nk_ctx* ctx, float* out_ms);            /* second event + synchronise */
/* FMA throughput of the device measured with a register-resident loop (TFLOP/s, 2 flops per FMA): the roofline
 * denominator for the FMA-bound kernels (F32 stencil, F64 convolution, double-evaluated activations). */
int nk_measure_fma_peak(nk_ctx* ctx, int32_t dtype, double* out_tflops);

/* Operations Min / Max: replaces CLReduce (J/backend/main/operations/linear/internal/opencl/CLReduce.java:34-147) with
 * the CPU implementation's semantics (J/backend/main/operations/other/internal/CPUReduce.java:72-140): writes ONE int, the
 * flat index of the smallest (want_max = 0) or largest element of the view, to element out_index of an I32 buffer.
 * Strict comparison: among equal extremes the lowest index wins. A NaN is never selected unless all elements are NaN
 * (the reference's choice then depends on its 64-element tiling). F32 / F64, fewer than 2^31 elements. */
int nk_arg_reduce(nk_ctx* ctx, int32_t want_max, int32_t dtype, int32_t rank, nk_buf* src, const int32_t* cfg, nk_buf* out_i32, int64_t out_index);

/* ---- fused elementwise expressions, compiled at run time ----
 * Counterpart of the kernels the reference generates for Device.optimizedOperationOf(Function, name)
 * (src/main/java/neureka/devices/Device.java:216-241; model: src/main/java/neureka/devices/opencl/utility/CLFunctionCompiler.java:47-196), plus
 * broadcasting, which the reference's compiler does not do. `expr` is one C expression of type T over x0 .. x5 built from
 *   op_add(a,b) op_sub op_mul op_div op_mod op_pow      the six Operator ops, forward
 *   f_<id>(a), df_<id>(a)                               the 23 functions of nk_fun and their derivatives (f_tanh, df_relu ...)
 *   T(<number>)                                         a constant in the tensor's type
 * e.g. "f_tanh(op_add(op_mul(x0,x1),x1))". Every operator rounds to the tensor's type and the scalar functions are the
 * ones the separate kernels use, so the result equals the op-by-op evaluation bit for bit. Operand extents must equal the
 * drain's or be 1 (broadcast). Needs libnvrtc.so.12 at run time (NK_ERR_UNSUPPORTED if absent); a malformed expression
 * gives NK_ERR_BAD_ARG with the compiler's log in nk_last_error. */
typedef struct nk_fused nk_fused;
int nk_fused_compile(nk_ctx* ctx, int32_t dtype, int32_t n_inputs, const char* expr, nk_fused** out);
int nk_fused_run(nk_ctx* ctx, nk_fused* f, int32_t rank, nk_buf* drn, const int32_t* cfg0,
                 nk_buf* const* srcs, const int32_t* const* cfgs);
int nk_fused_free(nk_fused* f);
/* The backward pass of such an expression w.r.t. input `target`, the sum over the dims that input is broadcast along
 * included: one kernel that recomputes the expression per element of the full index space, multiplies the error through
 * it and reduces -- no result-sized intermediate is read or written. The reference's compiler produces derivative kernels
 * too (src/main/java/neureka/devices/opencl/utility/CLFunctionCompiler.java:114, :155-157: a second kernel for `getDerivative(d)`); the reduction is this library's.
 * `terms` is a list of C statements over e (the error element) and x0 .. x5 that assigns term[0] .. term[n_leaves-1], one
 * per occurrence of the input in the expression, built from the forward vocabulary plus dop_div(d,a,b), dop_mod, dop_pow
 * (local derivative of the operator w.r.t. operand d), e.g. for tanh(x0*x1+x1) and target 1:
 *   "const T t0 = op_mul(x0,x1); const T t1 = op_add(t0,x1); const T t2 = op_mul(e, df_tanh(t1)); term[0] = t2;
 *    term[1] = op_mul(x0, t2);"
 * Every occurrence is summed separately, lowest reduced dim fastest (the order of nk_broadcast with d >= 0), and the
 * sums are added in occurrence order: where the op-by-op backward pass reduces at a single node of the expression the
 * result equals it bit for bit. `err` is result-shaped or a single (virtual) value; `grad` has the input's shape. */
int nk_fused_compile_grad(nk_ctx* ctx, int32_t dtype, int32_t n_inputs, int32_t target, int32_t n_leaves, const char* terms, nk_fused** out);
int nk_fused_run_grad(nk_ctx* ctx, nk_fused* f, int32_t rank, nk_buf* grad, const int32_t* cfg_grad, nk_buf* err, const int32_t* cfg_err,
                      nk_buf* const* srcs, const int32_t* const* cfgs);

/* ---- ordering between contexts (no reference counterpart: OpenCLDevice owns a single in-order queue) ----
 * A second nk_ctx on the same device is a second stream. An event recorded on one context's stream can be waited
 * for by another's, e.g. to let copies of finished results run beside the next computation. Waiting for an event
 * that was never recorded does not block. */
typedef struct nk_event nk_event;
int nk_event_create(nk_ctx* ctx, nk_event** out);
int nk_event_record(nk_ctx* ctx, nk_event* ev);          /* on ctx's stream, after the work queued so far */
int nk_stream_wait_event(nk_ctx* ctx, nk_event* ev);     /* work queued on ctx's stream from now on waits for ev */
int nk_event_free(nk_event* ev);

/* Failure-path check (no reference counterpart): runs the bounded mbarrier wait of the pipelined kernels on a barrier
 * that nothing completes, with the given limit (at most 1 s). The kernel returns by itself; the expired wait is then
 * reported by the next nk_sync / nk_read as NK_ERR_TIMEOUT, exactly as for a convolution kernel. */
int nk_probe_wait_timeout(nk_ctx* ctx, uint64_t limit_ns, uint64_t* out_waited_ns);

/* ---- multi-GPU (no reference counterpart: the reference has no multi-device execution) ----
 * (a) One process per GPU. A rank exports a buffer; peers open it and use it as the drain of nk_conv, so a
 * slab's results are stored straight into the owner's memory over NVLink (plain stores). */
#define NK_IPC_HANDLE_BYTES 64
int nk_ipc_export(nk_ctx* ctx, nk_buf* buf, uint8_t handle[NK_IPC_HANDLE_BYTES]);
int nk_ipc_open(nk_ctx* ctx, const uint8_t handle[NK_IPC_HANDLE_BYTES], int32_t dtype, int64_t n_elems, nk_buf** out);

/* (b) One process, several GPUs: the way a JVM holds several Device objects (J/devices/Device.java:259-279; the
 * backend extension hands them out, J/backend/api/BackendExtension.java:15-70). nk_group_open opens one context per
 * ordinal and enables peer access between the members once (the same ordinal twice = one GPU, two streams).
 * nk_group_ctx gives a member's context for the ordinary calls (alloc, write, kernels). */
typedef struct nk_group nk_group;
int nk_group_open(const int32_t* ordinals, int32_t n, nk_group** out);
int nk_group_size(nk_group* grp, int32_t* out_n);
int nk_group_ctx(nk_group* grp, int32_t member, nk_ctx** out_ctx);
int nk_group_close(nk_group* grp);
/* The split of `out_extent` output indices over `parts` members with `halo` extra input indices each (host
 * arithmetic only): member g computes outputs [out_lo[g], out_lo[g] + out_len[g]) from inputs
 * [in_lo[g], in_lo[g] + in_len[g]). Near-equal contiguous parts, the remainder to the first members. */
int nk_group_plan_slabs(int64_t out_extent, int32_t parts, int64_t halo, int64_t* out_lo, int64_t* out_len, int64_t* in_lo, int64_t* in_len);
/* Forward convolution image x kernel cut along output dim split_dim (image extent > kernel extent there): slabs[g] is
 * member g's dense input slab (the image's shape with in_len[g] along split_dim, on member g's device), kernels[g] its
 * copy of the kernel, `out` the full result on the FIRST member's device. Member 0 convolves into place; the others
 * convolve into a local slab and push it into `out` over NVLink on a second stream (overlapping the next call); the
 * first member's stream waits for the pushes, so work queued on it afterwards sees the assembled result. */
int nk_conv_sharded(nk_group* grp, int32_t dtype, int32_t rank, const int64_t* image_shape, const int64_t* kernel_shape, int32_t split_dim,
                    nk_buf* const* slabs, nk_buf* const* kernels, nk_buf* out);

/* ---- synthetic inputs: java.util.Random-compatible streams (host side) ----
 * Constants and polar Gaussian as J/backend/main/implementations/elementwise/CPURandomization.java:12-15, :265-284.
 * dist 0: uniform lo + (hi-lo)*next{Float|Double}(); dist 1: p0 + p1*nextGaussian(). One stream per call,
 * row-major element order. */
int nk_jrand_fill(int32_t dtype, int32_t dist, int64_t seed, double p0, double p1, void* host_out, int64_t n);
/* The same stream entered at element `start` (uniform only: the generator is jumped ahead), so that a rank can
 * generate just its own slab of a large tensor. */
int nk_jrand_fill_at(int32_t dtype, int32_t dist, int64_t seed, double p0, double p1, int64_t start,
                     void* host_out, int64_t n);

#ifdef __cplusplus
}
#endif
#endif /* NEUREKA_CUDA_H */
