// In-process device group: several GPUs of one box driven from ONE host process, the way a JVM holds several Device
// objects (src/main/java/neureka/devices/Device.java:259-279, BackendExtension.find, backend/api/BackendExtension.java:15-70).
// The reference itself never runs one operation on more than one device; this group adds exactly one such operation, the
// halo-split forward convolution: a large `x` call is cut along an output dim in which the image is larger than the kernel,
// device g computes output indices [lo_g, hi_g) of that dim from input indices [lo_g, hi_g + halo) -- its slab plus a halo of
// (kernel extent - 1) -- and the result is assembled in the memory of the group's first device.
//
// Data movement. Nothing is exchanged while computing: every device holds its input slab (with halo) and a copy of the
// kernel. Device 0 convolves straight into its rows of the result. Every other device convolves into a local slab and then
// pushes it into its rows of the result with device-to-device copies over NVLink on a second stream of its own
// (cudaMemcpyPeerAsync, one contiguous piece per outer index), so the push of one call overlaps the convolution of the
// next; two local slabs rotate. The result's owner stream waits on the push events: work queued on device 0 after
// nk_conv_sharded (a read, the next kernel) sees the assembled tensor. Peer memory is only ever written, by copy engines;
// no kernel of this library loads from another GPU.
#include <vector>

#include "nk_internal.h"
#include <cstring>

struct nk_group {
    std::vector<nk_ctx*> ctx;          // one context (= compute stream) per member
    std::vector<cudaStream_t> push;    // second stream per member for the assemble copies
    std::vector<cudaEvent_t> ev_conv[2], ev_push[2];
    std::vector<nk_buf*> local[2];     // rotating local result slabs of members 1..n-1
    std::vector<int64_t> local_elems;
    uint64_t calls = 0;
    uint32_t magic = 0x4e4b4750;       // 'NKGP'
};

extern "C" int nk_group_plan_slabs(int64_t out_extent, int32_t parts, int64_t halo, int64_t* out_lo, int64_t* out_len, int64_t* in_lo,
                                   int64_t* in_len) {
    // contiguous, near-equal slabs of the split output dim; earlier members take the remainder; members beyond the
    // extent get an empty slab
    if (out_extent < 1 || parts < 1 || halo < 0 || !out_lo || !out_len || !in_lo || !in_len) return NK_ERR_BAD_ARG;
    const int64_t base = out_extent / parts, rem = out_extent % parts;
    int64_t lo = 0;
    for (int g = 0; g < parts; g++) {
        const int64_t n = base + (g < rem ? 1 : 0);
        out_lo[g] = lo; out_len[g] = n;
        in_lo[g] = lo; in_len[g] = n > 0 ? n + halo : 0;
        lo += n;
    }
    return NK_OK;
}

extern "C" int nk_group_open(const int32_t* ordinals, int32_t n, nk_group** out) {
    if (!out) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_open: out pointer is null");
    *out = nullptr;
    if (!ordinals || n < 1 || n > 64) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_open: 1..64 device ordinals expected");
    nk_group* g = new (std::nothrow) nk_group();
    if (!g) return nk_fail(nullptr, NK_ERR_OOM, "nk_group_open: host allocation failed");
    int st = NK_OK;
    for (int i = 0; i < n && st == NK_OK; i++) {
        nk_ctx* c = nullptr;
        st = nk_device_open(ordinals[i], &c);
        if (st == NK_OK) g->ctx.push_back(c);
    }
    // every member may write into every other member's memory (the assemble); the same ordinal twice is one GPU with
    // two streams and needs nothing
    for (int i = 0; i < n && st == NK_OK; i++) {
        for (int j = 0; j < n && st == NK_OK; j++) {
            if (ordinals[i] == ordinals[j]) continue;
            int can = 0;
            cudaError_t e = cudaDeviceCanAccessPeer(&can, ordinals[i], ordinals[j]);
            if (e != cudaSuccess || !can) { st = nk_fail(nullptr, NK_ERR_UNSUPPORTED, "nk_group_open: device %d cannot reach device %d's memory", ordinals[i], ordinals[j]); break; }
            cudaSetDevice(ordinals[i]);
            e = cudaDeviceEnablePeerAccess(ordinals[j], 0);
            if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
            if (e != cudaSuccess) { st = nk_cuda_fail(nullptr, e, "cudaDeviceEnablePeerAccess"); break; }
            // Tensors come from device j's stream-ordered pool, which the call above does not cover: without this a copy
            // between members is staged through host memory (measured 30 GB/s instead of NVLink's 770)
            cudaMemPool_t pool = nullptr;
            e = cudaDeviceGetDefaultMemPool(&pool, ordinals[j]);
            if (e == cudaSuccess) {
                cudaMemAccessDesc desc;
                memset(&desc, 0, sizeof(desc));
                desc.location.type = cudaMemLocationTypeDevice;
                desc.location.id = ordinals[i];
                desc.flags = cudaMemAccessFlagsProtReadWrite;
                e = cudaMemPoolSetAccess(pool, &desc, 1);
            }
            if (e != cudaSuccess) st = nk_cuda_fail(nullptr, e, "cudaMemPoolSetAccess");
        }
    }
    for (int i = 0; i < n && st == NK_OK; i++) {
        cudaSetDevice(ordinals[i]);
        cudaStream_t s = nullptr;
        cudaError_t e = cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking);
        if (e == cudaSuccess) g->push.push_back(s);
        for (int r = 0; r < 2 && e == cudaSuccess; r++) {
            cudaEvent_t a = nullptr, b = nullptr;
            e = cudaEventCreateWithFlags(&a, cudaEventDisableTiming);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b, cudaEventDisableTiming);
            if (e == cudaSuccess) { g->ev_conv[r].push_back(a); g->ev_push[r].push_back(b); }
        }
        if (e != cudaSuccess) st = nk_cuda_fail(nullptr, e, "nk_group_open (streams and events)");
    }
    if (st != NK_OK) {
        nk_group_close(g);
        return st;
    }
    for (int r = 0; r < 2; r++) g->local[r].assign(size_t(n), nullptr);
    g->local_elems.assign(size_t(n), 0);
    *out = g;
    return NK_OK;
}

extern "C" int nk_group_size(nk_group* g, int32_t* out_n) {
    if (!g || g->magic != 0x4e4b4750 || !out_n) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_size: invalid group or null pointer");
    *out_n = int32_t(g->ctx.size());
    return NK_OK;
}

extern "C" int nk_group_ctx(nk_group* g, int32_t member, nk_ctx** out_ctx) {
    if (!g || g->magic != 0x4e4b4750 || !out_ctx) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_ctx: invalid group or null pointer");
    if (member < 0 || size_t(member) >= g->ctx.size()) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_ctx: member %d outside [0, %zu)", member, g->ctx.size());
    *out_ctx = g->ctx[size_t(member)];
    return NK_OK;
}

extern "C" int nk_group_close(nk_group* g) {
    if (!g) return NK_OK;
    if (g->magic != 0x4e4b4750) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_group_close: invalid group handle");
    for (size_t i = 0; i < g->ctx.size(); i++) {
        cudaSetDevice(g->ctx[i]->device);
        if (i < g->push.size()) { cudaStreamSynchronize(g->push[i]); }
        for (int r = 0; r < 2; r++) {
            if (i < g->local[r].size() && g->local[r][i]) nk_free(g->ctx[i], g->local[r][i]);
            if (i < g->ev_conv[r].size()) cudaEventDestroy(g->ev_conv[r][i]);
            if (i < g->ev_push[r].size()) cudaEventDestroy(g->ev_push[r][i]);
        }
        if (i < g->push.size()) cudaStreamDestroy(g->push[i]);
    }
    for (nk_ctx* c : g->ctx) nk_device_close(c);
    g->magic = 0;
    delete g;
    return NK_OK;
}

namespace {

// inline configuration [shape | strides | indicesMap | offset | spread] of a dense row-major tensor of `shape` ...
void dense_cfg(int rank, const int64_t* shape, int32_t* cfg) {
    int64_t st = 1;
    for (int k = rank - 1; k >= 0; k--) {
        cfg[k] = int32_t(shape[k]);
        cfg[rank + k] = int32_t(st);
        cfg[2 * rank + k] = int32_t(st);
        cfg[3 * rank + k] = 0;
        cfg[4 * rank + k] = 1;
        st *= shape[k];
    }
}
// ... and of the slice [lo, lo + len) along `dim` of a dense tensor of `parent` (parent strides, own row-major
// indicesMap, an offset on the split dim: what Neureka's slicing produces)
void slab_cfg(int rank, const int64_t* parent, int dim, int64_t lo, int64_t len, int32_t* cfg) {
    int64_t st = 1, im = 1;
    for (int k = rank - 1; k >= 0; k--) {
        const int64_t e = k == dim ? len : parent[k];
        cfg[k] = int32_t(e);
        cfg[rank + k] = int32_t(st);
        cfg[2 * rank + k] = int32_t(im);
        cfg[3 * rank + k] = k == dim ? int32_t(lo) : 0;
        cfg[4 * rank + k] = 1;
        st *= parent[k];
        im *= e;
    }
}

}  // namespace

extern "C" int nk_conv_sharded(nk_group* g, int32_t dtype, int32_t rank, const int64_t* image_shape, const int64_t* kernel_shape, int32_t split_dim,
                               nk_buf* const* slabs, nk_buf* const* kernels, nk_buf* out) {
    if (!g || g->magic != 0x4e4b4750) return nk_fail(nullptr, NK_ERR_BAD_ARG, "nk_conv_sharded: invalid group handle");
    nk_ctx* c0 = g->ctx[0];
    const int n = int(g->ctx.size());
    if (dtype != NK_F32 && dtype != NK_F64) return nk_fail(c0, NK_ERR_UNSUPPORTED, "nk_conv_sharded: dtype %d not supported (F32/F64 only)", dtype);
    if (rank < 1 || rank > NK_MAX_RANK || !image_shape || !kernel_shape || !slabs || !kernels || !out)
        return nk_fail(c0, NK_ERR_BAD_ARG, "nk_conv_sharded: bad rank or null argument");
    if (split_dim < 0 || split_dim >= rank || !(image_shape[split_dim] > kernel_shape[split_dim]))
        return nk_fail(c0, NK_ERR_BAD_ARG, "nk_conv_sharded: dim %d cannot be halo-split (the image must be larger than the kernel there)", split_dim);
    if (out->magic != 0x4e4b4246 || out->device != c0->device || out->dtype != dtype)
        return nk_fail(c0, NK_ERR_BAD_ARG, "nk_conv_sharded: the result buffer must live on the group's first device and have the call's dtype");
    int64_t out_shape[NK_MAX_RANK], total_out = 1;
    for (int k = 0; k < rank; k++) {
        const int64_t a = image_shape[k], b = kernel_shape[k];
        if (a < 1 || b < 1 || a >= (int64_t(1) << 31) || b >= (int64_t(1) << 31)) return nk_fail(c0, NK_ERR_BAD_ARG, "nk_conv_sharded: extent out of range in dim %d", k);
        out_shape[k] = (a > b ? a - b : b - a) + 1;
        total_out *= out_shape[k];
    }
    if (total_out > out->n_elems) return nk_fail(c0, NK_ERR_BOUNDS, "nk_conv_sharded: the result needs %lld elements, the buffer holds %lld", (long long)total_out, (long long)out->n_elems);
    if (total_out >= (int64_t(1) << 31)) return nk_fail(c0, NK_ERR_UNSUPPORTED, "nk_conv_sharded: results of 2^31 elements or more are not supported");
    const int64_t halo = kernel_shape[split_dim] - 1;
    const size_t nn = static_cast<size_t>(n);
    std::vector<int64_t> olo(nn), olen(nn), ilo(nn), ilen(nn);
    nk_group_plan_slabs(out_shape[split_dim], n, halo, olo.data(), olen.data(), ilo.data(), ilen.data());
    int64_t outer = 1, inner = 1;   // result elements before / after the split dim: a member's rows are `outer` contiguous pieces
    for (int k = 0; k < split_dim; k++) outer *= out_shape[k];
    for (int k = split_dim + 1; k < rank; k++) inner *= out_shape[k];
    const size_t es = nk_dtype_size(dtype);
    const int r = int(g->calls++ & 1);
    int32_t cfg_in[5 * NK_MAX_RANK], cfg_k[5 * NK_MAX_RANK], cfg_out[5 * NK_MAX_RANK];
    dense_cfg(rank, kernel_shape, cfg_k);
    for (int i = 0; i < n; i++) {
        if (olen[size_t(i)] == 0) continue;
        nk_ctx* c = g->ctx[size_t(i)];
        cudaError_t e = cudaSetDevice(c->device);
        if (e != cudaSuccess) return nk_cuda_fail(c0, e, "cudaSetDevice");
        int64_t local_in[NK_MAX_RANK], local_out[NK_MAX_RANK];
        for (int k = 0; k < rank; k++) { local_in[k] = image_shape[k]; local_out[k] = out_shape[k]; }
        local_in[split_dim] = ilen[size_t(i)];
        local_out[split_dim] = olen[size_t(i)];
        int64_t in_elems = 1;
        for (int k = 0; k < rank; k++) in_elems *= local_in[k];
        if (in_elems >= (int64_t(1) << 31))   // the views handed to nk_conv are the reference's int-sized configurations
            return nk_fail(c0, NK_ERR_UNSUPPORTED, "nk_conv_sharded: member %d's slab has %lld elements, 2^31 or more are not supported", i, (long long)in_elems);
        dense_cfg(rank, local_in, cfg_in);
        int st;
        if (i == 0) {
            slab_cfg(rank, out_shape, split_dim, olo[0], olen[0], cfg_out);   // the owner computes straight into place
            st = nk_conv(c, dtype, rank, out, cfg_out, slabs[0], cfg_in, kernels[0], cfg_k, -1);
            if (st) return nk_fail(c0, st, "nk_conv_sharded: member 0: %s", nk_last_error(c));
            continue;
        }
        const int64_t need = outer * olen[size_t(i)] * inner;
        for (int q = 0; q < 2; q++) {
            if (g->local[q][size_t(i)] && g->local_elems[size_t(i)] < need) { nk_free(c, g->local[q][size_t(i)]); g->local[q][size_t(i)] = nullptr; }
        }
        for (int q = 0; q < 2; q++) {
            if (!g->local[q][size_t(i)]) {
                st = nk_alloc(c, dtype, need, &g->local[q][size_t(i)]);
                if (st) return nk_fail(c0, st, "nk_conv_sharded: member %d: %s", i, nk_last_error(c));
            }
        }
        g->local_elems[size_t(i)] = need;
        nk_buf* loc = g->local[r][size_t(i)];
        // the push that last read this local slab must be done before it is overwritten
        e = cudaStreamWaitEvent(c->stream, g->ev_push[r][size_t(i)], 0);
        if (e != cudaSuccess) return nk_cuda_fail(c0, e, "cudaStreamWaitEvent");
        dense_cfg(rank, local_out, cfg_out);
        st = nk_conv(c, dtype, rank, loc, cfg_out, slabs[i], cfg_in, kernels[i], cfg_k, -1);
        if (st) return nk_fail(c0, st, "nk_conv_sharded: member %d: %s", i, nk_last_error(c));
        e = cudaEventRecord(g->ev_conv[r][size_t(i)], c->stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(g->push[size_t(i)], g->ev_conv[r][size_t(i)], 0);
        const int64_t piece = olen[size_t(i)] * inner;   // contiguous in both the local slab and the result
        for (int64_t o = 0; o < outer && e == cudaSuccess; o++) {
            char* dst = static_cast<char*>(out->ptr) + size_t((o * out_shape[split_dim] + olo[size_t(i)]) * inner) * es;
            const char* src = static_cast<const char*>(loc->ptr) + size_t(o * piece) * es;
            e = cudaMemcpyPeerAsync(dst, c0->device, src, c->device, size_t(piece) * es, g->push[size_t(i)]);
        }
        if (e == cudaSuccess) e = cudaEventRecord(g->ev_push[r][size_t(i)], g->push[size_t(i)]);
        if (e != cudaSuccess) return nk_cuda_fail(c0, e, "nk_conv_sharded (assemble copies)");
    }
    // the owner's stream sees the assembled result
    cudaError_t e = cudaSetDevice(c0->device);
    for (int i = 1; i < n && e == cudaSuccess; i++)
        if (olen[size_t(i)] > 0) e = cudaStreamWaitEvent(c0->stream, g->ev_push[r][size_t(i)], 0);
    if (e != cudaSuccess) return nk_cuda_fail(c0, e, "nk_conv_sharded (owner waits for the pushes)");
    return NK_OK;
}
