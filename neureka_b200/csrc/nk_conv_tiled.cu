// Routing of forward convolutions to the tiled stencil family: eligibility test, plan construction, tensor-map
// encoding and the (KH, KW) dispatch. The kernels themselves are instantiated per dtype / loader / rows-per-thread
// in nk_conv_tiled_inst_*.cu.

#include "nk_conv_wgrad.cuh"

int nk_wgrad_dispatch_f32(nk_ctx*, int, int, float*, WgradPlan&, const TmaImage&, const TmaImage&);
int nk_wgrad_dispatch_f64(nk_ctx*, int, int, double*, WgradPlan&, const TmaImage&, const TmaImage&);

#define NK_DECL(suf, ty)                                                                                                   \
    int nk_tiled_dispatch_##suf##_ldgsts(nk_ctx*, int, int, ty*, const ty*, const ty*, TiledPlan&, const TmaImage*);       \
    int nk_tiled_dispatch_##suf##_tma4(nk_ctx*, int, int, ty*, const ty*, const ty*, TiledPlan&, const TmaImage*);         \
    int nk_tiled_dispatch_##suf##_tma8(nk_ctx*, int, int, ty*, const ty*, const ty*, TiledPlan&, const TmaImage*);
NK_DECL(f32, float)
NK_DECL(f64, double)

namespace {

bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            cudaGetLastError();
    }
    return fn;
}

}  // namespace

// -1: this view cannot be described by a tensor map (the caller uses the LDGSTS loader); otherwise a status.
int nk_tma_encode(nk_ctx* ctx, int dtype, const TmaImage& img, int box_w, int box_h, bool has_y, CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    cuuint64_t dims[5], strides[4];
    cuuint32_t box[5], estr[5];
    for (int k = 0; k < img.nd; k++) {
        dims[k] = img.dims[k];
        box[k] = 1;
        estr[k] = 1;
        if (k > 0) strides[k - 1] = img.strides_bytes[k];
    }
    box[0] = cuuint32_t(box_w);
    if (has_y) box[1] = cuuint32_t(box_h);
    CUresult r = fn(out, dtype == NK_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT64, cuuint32_t(img.nd),
                    const_cast<void*>(img.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
    return NK_OK;
}

// A dense 2-D F32 array [rows, cols] (row pitch in bytes, a multiple of 16) as a tensor map with a box of box_cols x
// box_rows elements and the given shared-memory swizzle (0 none, 1 = 32 B, 2 = 64 B, 3 = 128 B). -1 when the driver's
// encoder is missing or refuses.
int nk_tma_encode_2d_f32(const void* base, uint64_t rows, uint64_t cols, uint64_t pitch_bytes, int box_cols, int box_rows, int swizzle,
                         CUtensorMap* out) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    cuuint64_t dims[2] = {cols, rows}, strides[1] = {pitch_bytes};
    cuuint32_t box[2] = {cuuint32_t(box_cols), cuuint32_t(box_rows)}, estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : swizzle == 2 ? CU_TENSOR_MAP_SWIZZLE_64B
                                : swizzle == 1 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? NK_OK : -1;
}

// Tensor map description of a whole view: X, optionally Y, then the outer dims (innermost first). False when the
// view cannot be described (unaligned base, strides that are not positive multiples of 16 bytes).
static bool nk_describe_for_tma(const nk_buf* buf, const NkView& v, size_t es, bool has_y, int n_outer, TmaImage* img) {
    const int rank = v.rank, X = rank - 1, Y = rank - 2;
    const char* base = static_cast<const char*>(buf->ptr) + v.base * int64_t(es);
    if (reinterpret_cast<uintptr_t>(base) % 16 || v.estride[X] != 1) return false;
    int n = 0;
    img->base = base;
    img->dims[n] = uint64_t(v.shape[X]); img->strides_bytes[n] = es; n++;
    if (has_y) {
        if (v.estride[Y] <= 0 || (v.estride[Y] * int64_t(es)) % 16) return false;
        img->dims[n] = uint64_t(v.shape[Y]); img->strides_bytes[n] = uint64_t(v.estride[Y]) * es; n++;
    }
    for (int k = n_outer - 1; k >= 0; k--) {
        const int64_t ext = v.shape[k], st = v.estride[k];
        img->dims[n] = uint64_t(ext);
        if (ext == 1) {
            uint64_t prev = img->strides_bytes[n - 1] * img->dims[n - 1];
            img->strides_bytes[n] = ((prev + 15) / 16) * 16;
            if (img->strides_bytes[n] == 0) img->strides_bytes[n] = 16;
        } else {
            if (st <= 0 || (st * int64_t(es)) % 16 || uint64_t(st) * es >= (uint64_t(1) << 40)) return false;
            img->strides_bytes[n] = uint64_t(st) * es;
        }
        n++;
    }
    img->nd = n;
    return n >= 2 && n <= 5;
}

// ---- staging of operands a tensor map cannot describe ----------------------------------------------------------------
// A tensor map wants a 16-byte aligned base and strides that are multiples of 16 bytes; a tensor of, say, 126 floats per row
// has neither. Such an operand of a deconvolution is copied once into a dense block whose rows are padded to 16 bytes and
// the TMA kernels read the copy: for the error tensor of an image gradient that is 1/channels of the traffic, against a
// fallback to the gather family that measured 20 times slower. The block comes from the device's stream-ordered pool:
// copy, kernel and release all queue on the context's stream.
struct StageDims {
    int rank;
    long long total, base;
    long long div[NK_MAX_RANK], sstride[NK_MAX_RANK], dstride[NK_MAX_RANK];
};
template <class T>
__global__ void __launch_bounds__(256) nk_stage_kernel(T* __restrict__ dst, const T* __restrict__ src, StageDims d) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < d.total; i += stride) {
        long long rem = i, so = d.base, dof = 0;
        for (int k = 0; k < d.rank; k++) {
            const long long idx = rem / d.div[k];
            rem -= idx * d.div[k];
            so += idx * d.sstride[k];
            dof += idx * d.dstride[k];
        }
        dst[dof] = src[so];
    }
}
struct Staged {
    nk_buf buf;     // stands in for the operand's handle (pointer, dtype, device)
    NkView view;    // dense, rows padded to 16 bytes, base 0
    bool used = false;
};
static int nk_stage_operand(nk_ctx* ctx, int dtype, const nk_buf* src, const NkView& v, Staged* out) {
    const size_t es = nk_dtype_size(dtype);
    const int rank = v.rank, X = rank - 1;
    const int64_t cw = int64_t(16 / es);
    const int64_t pitch = ((v.shape[X] + cw - 1) / cw) * cw;
    StageDims d;
    memset(&d, 0, sizeof(d));
    d.rank = rank;
    d.base = v.base;
    out->view = v;
    out->view.base = 0;
    int64_t ds = 1, dv = 1;
    for (int k = rank - 1; k >= 0; k--) {
        d.div[k] = dv;
        dv *= v.shape[k];
        d.sstride[k] = v.estride[k];
        d.dstride[k] = ds;
        out->view.estride[k] = ds;
        ds *= (k == X) ? pitch : v.shape[k];
    }
    d.total = dv;
    out->view.dense_row_major = pitch == v.shape[X];
    if (ds >= (int64_t(1) << 40)) return -1;
    void* ptr = nullptr;
    cudaError_t e = cudaMallocAsync(&ptr, size_t(ds) * es, ctx->stream);
    if (e != cudaSuccess) { cudaGetLastError(); return -1; }   // no room for a copy: the caller falls back to another family
    out->buf = *src;
    out->buf.ptr = ptr;
    out->buf.n_elems = ds;
    out->buf.owned = false;
    out->used = true;
    const int grid = nk_grid_for(ctx, d.total, 256, 16);
    if (dtype == NK_F32) nk_stage_kernel<float><<<grid, 256, 0, ctx->stream>>>(static_cast<float*>(ptr), static_cast<const float*>(src->ptr), d);
    else nk_stage_kernel<double><<<grid, 256, 0, ctx->stream>>>(static_cast<double*>(ptr), static_cast<const double*>(src->ptr), d);
    return nk_after_launch(ctx, "nk_stage_kernel");
}
static void nk_stage_release(nk_ctx* ctx, Staged* s) {
    if (s->used) cudaFreeAsync(s->buf.ptr, ctx->stream);
    s->used = false;
}

// Deconvolution (d >= 0) whose result is the small, kernel-like tensor: D[p] = sum_q T1[p+q] * T2[q] in every dim
// (the drain is not larger than T1 anywhere), the last one or two dims being a window of few taps over large planes.
static int nk_wgrad_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                        nk_buf* s2, const NkView& v2, bool* handled) {
    if (ctx->conv_path == NK_CONV_TILED) return NK_OK;
    const int rank = v0.rank, X = rank - 1, Y = rank - 2;
    if (rank < 2 || !v0.imap_row_major) return NK_OK;
    for (int k = 0; k < rank; k++)
        if (v0.shape[k] > v1.shape[k]) return NK_OK;          // tau = p + q everywhere
    const int64_t KW = v0.shape[X];
    if (v2.shape[X] < 64 || KW > 9) return NK_OK;             // a real plane to reduce over, a real window
    bool has_y = v0.shape[Y] <= 7 && v2.shape[Y] > 1;
    int64_t KH = has_y ? v0.shape[Y] : 1;
    const int n_outer = has_y ? rank - 2 : rank - 1;
    if (n_outer > 3) return NK_OK;
    // long reductions only: otherwise the generic family is as good
    int64_t terms = 1;
    for (int k = 0; k < rank; k++) terms *= v2.shape[k];
    if (terms < 65536) return NK_OK;
    WgradPlan p;
    memset(&p, 0, sizeof(p));
    p.n_outer = n_outer;
    p.has_y = has_y ? 1 : 0;
    p.NP = 1; p.NQ = 1;
    for (int k = 0; k < n_outer; k++) {
        p.oext[k] = v0.shape[k]; p.os[k] = v0.estride[k];
        p.qext[k] = v2.shape[k];
        p.NP *= v0.shape[k];
        p.NQ *= v2.shape[k];
    }
    p.EW = int(v2.shape[X]);
    p.EH = has_y ? int(v2.shape[Y]) : 1;
    p.sDx = v0.estride[X];
    p.sDy = has_y ? v0.estride[Y] : 0;
    p.bD = v0.base;
    const size_t es = nk_dtype_size(dtype);
    TmaImage imgA, imgE;
    Staged stA, stE;
    bool ok = true;
    if (!nk_describe_for_tma(s1, v1, es, has_y, n_outer, &imgA)) {
        const int sst = nk_stage_operand(ctx, dtype, s1, v1, &stA);
        if (sst > 0) return sst;
        ok = sst == 0 && nk_describe_for_tma(&stA.buf, stA.view, es, has_y, n_outer, &imgA);
    }
    if (ok && !nk_describe_for_tma(s2, v2, es, has_y, n_outer, &imgE)) {
        const int sst = nk_stage_operand(ctx, dtype, s2, v2, &stE);
        if (sst > 0) { nk_stage_release(ctx, &stA); return sst; }
        ok = sst == 0 && nk_describe_for_tma(&stE.buf, stE.view, es, has_y, n_outer, &imgE);
    }
    int st = -1;
    if (ok) {
        p.nd = imgA.nd;
        st = (dtype == NK_F32) ? nk_wgrad_dispatch_f32(ctx, int(KH), int(KW), (float*)drn->ptr, p, imgA, imgE)
                               : nk_wgrad_dispatch_f64(ctx, int(KH), int(KW), (double*)drn->ptr, p, imgA, imgE);
    }
    nk_stage_release(ctx, &stA);
    nk_stage_release(ctx, &stE);
    if (st == -1) return NK_OK;
    if (st != NK_OK) return st;
    ctx->last_conv_path = NK_CONV_TMA;
    *handled = true;
    return NK_OK;
}

// Deconvolution (d >= 0) whose result is the larger, image-like tensor -- the gradient of a convolution w.r.t. its
// image: D[p] = sum_t T1[t] * T2[p - t] in the sliding dims. Rewritten as a correlation of the zero-padded error T2
// with the flipped weights T1, it runs on the same TMA kernel: tile loads start s1-1 elements before the output
// coordinate (the tensor map returns zeros outside T2, which is exactly the reference's "no such term"), and the
// weights are staged back to front through negative kernel strides. Outer dims may be batch-like (T1 extent 1: T2
// follows the output index), flipped outer windows, or follow T1 (T2 extent 1, e.g. the channels of the image).
static int nk_deconv_tiled_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                               nk_buf* s2, const NkView& v2, bool* handled) {
    if (ctx->conv_path == NK_CONV_TILED) return NK_OK;      // the padded form needs the tensor map's zero fill
    const int rank = v0.rank;
    const int X = rank - 1;
    if (!v0.imap_row_major || rank < 2) return NK_OK;
    {
        int st = nk_wgrad_try(ctx, dtype, drn, v0, s1, v1, s2, v2, handled);
        if (st || *handled) return st;
    }
    NkView vi = v2;          // image = T2 (the error); replaced by a padded copy below if a tensor map cannot describe it
    const void* iptr = s2->ptr;
    const NkView& vk = v1;   // weights = T1
    if (v0.estride[X] != 1) return NK_OK;
    // sliding dim X: tau = p - q (drain larger than T1), window of s1 taps
    if (!(v0.shape[X] > vk.shape[X])) return NK_OK;
    const int64_t KW = vk.shape[X];
    if (v0.shape[X] < 16) return NK_OK;
    int n_outer = rank - 1;
    int64_t KH = 1;
    bool has_y = false;
    const int Y = rank - 2;
    if (v0.shape[Y] > vk.shape[Y] && vk.shape[Y] <= 7 && v0.shape[Y] > 1 && vi.shape[Y] > 1) { has_y = true; KH = vk.shape[Y]; n_outer = rank - 2; }
    if (n_outer > 3 || 1 + (has_y ? 1 : 0) + n_outer > 5) return NK_OK;
    const size_t es = nk_dtype_size(dtype);
    const int CW = int(16 / es);
    Staged staged;
    {
        bool describable = vi.estride[X] == 1 && (reinterpret_cast<uintptr_t>(static_cast<const char*>(iptr) + vi.base * int64_t(es)) % 16) == 0;
        for (int k = 0; k < X && describable; k++)
            if (vi.shape[k] > 1 && (vi.estride[k] <= 0 || (vi.estride[k] * int64_t(es)) % 16)) describable = false;
        if (!describable) {
            // only worth a copy if the window is one the tiled family is instantiated for; the dispatch below decides, and a
            // wasted copy of the (small) error tensor is cheap next to the gather family it falls back to
            const int sst = nk_stage_operand(ctx, dtype, s2, v2, &staged);
            if (sst > 0) return sst;
            if (sst < 0) return NK_OK;
            vi = staged.view;
            iptr = staged.buf.ptr;
        }
    }
    TiledPlan p;
    TmaImage img;
    // Builds the plan. with_wloop: outer dims in which the drain follows T1 while T2 has extent 1 (the output channels of
    // an image gradient: they select weights and a drain plane, nothing else) are taken out of the tile index and become
    // the weight loop of a chunk -- one tile load then feeds all of them.
    auto build = [&](bool with_wloop) -> bool {
        memset(&p, 0, sizeof(p));
        p.has_y = has_y ? 1 : 0;
        p.NP = 1;
        int64_t NQ = 1;
        int64_t bK = vk.base;
        int no = 0;
        int kept[NK_MAX_RANK];
        for (int k = 0; k < n_outer; k++) {
            const int64_t e0 = v0.shape[k], e1 = vk.shape[k], e2 = vi.shape[k];
            if (with_wloop && !(e0 > e1) && e2 == 1 && e0 > 1) {
                if (e0 + e2 - 1 > e1) return false;
                p.wext[p.n_w] = e0; p.wos[p.n_w] = v0.estride[k]; p.wK[p.n_w] = vk.estride[k];
                p.n_w++;
                continue;
            }
            kept[no] = k;
            p.oext[no] = e0; p.os[no] = v0.estride[k];
            if (e0 > e1) {
                // tau = p - q: flipped window of e1 taps over T2 starting at p - (e1 - 1); e1 == 1 is the batch-like case
                p.qext[no] = e1; p.pI[no] = vi.estride[k]; p.qI[no] = vi.estride[k];
                p.pK[no] = 0; p.qK[no] = -vk.estride[k];
                bK += (e1 - 1) * vk.estride[k];
                p.padO[no] = int(e1 - 1);
            } else {
                // tau = p + q, q over T2: only the consistent case p + q < e1 for every p, q is taken here
                if (e0 + e2 - 1 > e1) return false;
                p.qext[no] = e2; p.pI[no] = 0; p.qI[no] = vi.estride[k];
                p.pK[no] = vk.estride[k]; p.qK[no] = vk.estride[k];
                p.padO[no] = 0;
            }
            if (p.qext[no] > 65535) return false;
            p.NP *= e0;
            NQ *= p.qext[no];
            no++;
        }
        p.n_outer = no;
        if (NQ > 4096) return false;
        p.NQ = int(NQ);
        p.wloop = (with_wloop && p.n_w > 0 && NQ == 1) ? 1 : 0;
        if (with_wloop && !p.wloop) return false;
        if (vi.shape[X] > 0x3fffffff || v0.shape[X] > 0x3fffffff) return false;
        p.IW = int(vi.shape[X]); p.OW = int(v0.shape[X]);
        p.padX = int(KW - 1);
        p.xoff = (CW - p.padX % CW) % CW;
        p.sKx = -vk.estride[X];
        bK += (KW - 1) * vk.estride[X];
        if (has_y) {
            p.IH = int(vi.shape[Y]); p.OH = int(v0.shape[Y]);
            p.padY = int(KH - 1);
            p.sIy = vi.estride[Y]; p.sOy = v0.estride[Y];
            p.sKy = -vk.estride[Y];
            bK += (KH - 1) * vk.estride[Y];
        } else {
            p.IH = 1; p.OH = 1;
        }
        p.bI = vi.base; p.bK = bK; p.bO = v0.base;
        p.vec = 0;
        bool vec_out = p.xoff == 0 && aligned_to(drn->ptr, 16) && (p.bO % CW == 0) && (p.sOy % CW == 0);
        for (int k = 0; k < no; k++)
            if (p.os[k] % CW) vec_out = false;
        for (int k = 0; k < p.n_w; k++)
            if (p.wos[k] % CW) vec_out = false;
        p.vec_out = vec_out ? 1 : 0;

        // tensor map over T2 (the dims of the tile index only)
        if (!aligned_to(static_cast<const char*>(iptr) + p.bI * int64_t(es), 16)) return false;
        int n = 0;
        img.base = static_cast<const char*>(iptr) + p.bI * int64_t(es);
        img.dims[n] = uint64_t(p.IW); img.strides_bytes[n] = es; n++;
        if (has_y) {
            if (p.sIy <= 0 || (p.sIy * int64_t(es)) % 16) return false;
            img.dims[n] = uint64_t(p.IH); img.strides_bytes[n] = uint64_t(p.sIy) * es; n++;
        }
        for (int j = no - 1; j >= 0; j--) {
            const int k = kept[j];
            const int64_t ext = vi.shape[k], st = vi.estride[k];
            img.dims[n] = uint64_t(ext);
            if (ext == 1) {
                uint64_t prev = img.strides_bytes[n - 1] * img.dims[n - 1];
                img.strides_bytes[n] = ((prev + 15) / 16) * 16;
                if (img.strides_bytes[n] == 0) img.strides_bytes[n] = 16;
            } else {
                if (st <= 0 || (st * int64_t(es)) % 16 || uint64_t(st) * es >= (uint64_t(1) << 40)) return false;
                img.strides_bytes[n] = uint64_t(st) * es;
            }
            n++;
        }
        if (n < 2 || n > 5) return false;
        img.nd = n;
        p.tma_nd = n;
        return true;
    };
    auto dispatch = [&]() -> int {
        if (dtype == NK_F32) return nk_tiled_dispatch_f32_tma4(ctx, int(KH), int(KW), (float*)drn->ptr, (const float*)iptr, (const float*)s1->ptr, p, &img);
        return nk_tiled_dispatch_f64_tma4(ctx, int(KH), int(KW), (double*)drn->ptr, (const double*)iptr, (const double*)s1->ptr, p, &img);
    };
    int st = -1;
    if (has_y && build(true)) st = dispatch();          // the weight loop first; -1 = it does not apply (sets too large, no persistent walk)
    if (st == -1 && build(false)) st = dispatch();
    nk_stage_release(ctx, &staged);
    if (st == -1) return NK_OK;
    if (st != NK_OK) return st;
    ctx->last_conv_path = NK_CONV_TMA;
    *handled = true;
    return NK_OK;
}
// Returns NK_OK with *handled = true when the call was launched on a tiled family, NK_OK with *handled = false
// when the views do not qualify (the caller then uses the generic family).
int nk_conv_tiled_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                      nk_buf* s2, const NkView& v2, int d, bool force, bool* handled) {
    *handled = false;
    if (d >= 0) return nk_deconv_tiled_try(ctx, dtype, drn, v0, s1, v1, s2, v2, handled);
    const int rank = v0.rank;
    const int X = rank - 1;
    if (!v0.imap_row_major) return NK_OK;
    // which operand is the image: the one that is larger along X
    const bool img_first = v1.shape[X] >= v2.shape[X];
    const NkView& vi = img_first ? v1 : v2;
    const NkView& vk = img_first ? v2 : v1;
    nk_buf* bi = img_first ? s1 : s2;
    nk_buf* bk = img_first ? s2 : s1;
    if (vi.estride[X] != 1 || v0.estride[X] != 1) return NK_OK;
    const int64_t KW = vk.shape[X];
    const int64_t OW = vi.shape[X] - KW + 1;
    if (v0.shape[X] != OW) return NK_OK;
    if (!force && OW < 16) return NK_OK;   // too narrow to fill a warp's row segment
    // the second-to-last dim slides too when it is a small window of the same operand; otherwise it is an
    // outer dim like all the others and the tile height is 1 row of work
    int n_outer = rank - 1;
    int64_t KH = 1, IH = 1, OH = 1, sIy = 0, sKy = 0, sOy = 0;
    bool has_y = false;
    if (rank >= 2) {
        const int Y = rank - 2;
        const bool window_y = vi.shape[Y] >= vk.shape[Y] && vk.shape[Y] <= 7 && vi.shape[Y] > 1;
        if (window_y) {
            KH = vk.shape[Y]; IH = vi.shape[Y]; OH = IH - KH + 1;
            if (v0.shape[Y] != OH) return NK_OK;
            sIy = vi.estride[Y]; sKy = vk.estride[Y]; sOy = v0.estride[Y];
            n_outer = rank - 2;
            has_y = true;
        }
    }
    if (n_outer > NK_TILED_MAX_OUTER) return NK_OK;
    TiledPlan p;
    memset(&p, 0, sizeof(p));
    p.n_outer = n_outer;
    p.has_y = has_y ? 1 : 0;
    p.NP = 1;
    int64_t NQ = 1;
    for (int k = 0; k < n_outer; k++) {
        const int64_t a = vi.shape[k], b = vk.shape[k], o = v0.shape[k];
        const int64_t n = a < b ? a : b, big = a < b ? b : a;
        if (o + n - 1 > big) return NK_OK;            // inconsistent drain: let the generic path report it
        if (a == b && o != 1) return NK_OK;
        p.oext[k] = o; p.os[k] = v0.estride[k];
        p.qext[k] = n; p.qI[k] = vi.estride[k]; p.qK[k] = vk.estride[k];
        p.pI[k] = (a > b) ? vi.estride[k] : 0;
        p.pK[k] = (a < b) ? vk.estride[k] : 0;
        p.NP *= o;
        NQ *= n;
    }
    if (NQ > 4096) return NK_OK;
    p.NQ = int(NQ);
    if (vi.shape[X] > 0x3fffffff || IH > 0x3fffffff) return NK_OK;
    p.IH = int(IH); p.IW = int(vi.shape[X]); p.OH = int(OH); p.OW = int(OW);
    p.sIy = sIy; p.sKy = sKy; p.sKx = vk.estride[X]; p.sOy = sOy;
    p.bI = vi.base; p.bK = vk.base; p.bO = v0.base;

    const size_t es = nk_dtype_size(dtype);
    const int CW = int(16 / es);
    // 16-byte global->shared copies: every chunk address = ptr + (bI + outer strides + y*sIy + x0 + col) elements
    bool vec = aligned_to(bi->ptr, 16) && (p.bI % CW == 0) && (p.sIy % CW == 0);
    bool vec_out = aligned_to(drn->ptr, 16) && (p.bO % CW == 0) && (p.sOy % CW == 0);
    for (int k = 0; k < n_outer; k++) {
        if (p.pI[k] % CW || p.qI[k] % CW) vec = false;
        if (p.os[k] % CW) vec_out = false;
    }
    p.vec = vec ? 1 : 0;
    p.vec_out = vec_out ? 1 : 0;
    p.remote_out = drn->ipc ? 1 : 0;

    // ---- can a tensor map describe the image view? (<= 5 dims, base and strides 16-byte aligned, positive) ----------
    TmaImage img;
    bool tma_ok = ctx->conv_path != NK_CONV_TILED && vec && (1 + (has_y ? 1 : 0) + n_outer) <= 5 && (1 + (has_y ? 1 : 0) + n_outer) >= 2;
    if (tma_ok) {
        int n = 0;
        img.base = static_cast<const char*>(bi->ptr) + p.bI * int64_t(es);
        img.dims[n] = uint64_t(p.IW); img.strides_bytes[n] = es; n++;
        if (has_y) { img.dims[n] = uint64_t(p.IH); img.strides_bytes[n] = uint64_t(p.sIy) * es; n++; if (p.sIy <= 0) tma_ok = false; }
        for (int k = n_outer - 1; k >= 0 && tma_ok; k--) {
            const int64_t ext = vi.shape[k], st = vi.estride[k];
            img.dims[n] = uint64_t(ext);
            if (ext == 1) {
                // the stride of an extent-1 dim is never applied; give the encoder a legal value
                uint64_t prev = img.strides_bytes[n - 1] * img.dims[n - 1];
                img.strides_bytes[n] = ((prev + 15) / 16) * 16;
                if (img.strides_bytes[n] == 0) img.strides_bytes[n] = 16;
            } else {
                if (st <= 0 || (st * int64_t(es)) % 16) tma_ok = false;
                img.strides_bytes[n] = uint64_t(st) * es;
            }
            if (p.qext[k] > 65535) tma_ok = false;
            n++;
        }
        img.nd = n;
        p.tma_nd = n;
        for (int k = 1; k < n && tma_ok; k++)
            if (img.strides_bytes[k] >= (uint64_t(1) << 40)) tma_ok = false;
    }

    int st = -1;
    const bool f32 = dtype == NK_F32;
    float* of = (float*)drn->ptr; const float* If = (const float*)bi->ptr; const float* Kf = (const float*)bk->ptr;
    double* od = (double*)drn->ptr; const double* Id = (const double*)bi->ptr; const double* Kd = (const double*)bk->ptr;
    int family = NK_CONV_TILED;
    if (tma_ok) {
        // 8 output rows per thread halve the shared-memory reads per multiply-add but double the work unit:
        // compare the two tilings by resident waves x relative tile time (32-row tiles are ~10 % less efficient)
        const int64_t slots = int64_t(ctx->prop.multiProcessorCount) * 2;
        const int tw = 32 * CW;
        const int64_t tiles8 = int64_t((p.OW + tw - 1) / tw) * ((p.OH + 63) / 64) * p.NP;
        const int64_t tiles4 = int64_t((p.OW + tw - 1) / tw) * ((p.OH + 31) / 32) * p.NP;
        const double cost8 = double((tiles8 + slots - 1) / slots) * 2.0;
        const double cost4 = double((tiles4 + slots - 1) / slots) * 1.1;
        // a drain on another GPU: results leave over NVLink as tiles finish, and the owner's link is the bottleneck of
        // an assemble -- short-lived tiles start that stream early and keep it steady
        // (only a short launch -- under two waves of tall tiles -- is dominated by that start-up; measured with 7 peers
        // storing into one owner: 0.198 ms against 0.227 ms; with more waves the tall tiles' efficiency wins again)
        // (with a tile per resident slot or more the launch is a balanced persistent walk: no wave rounding to compare)
        bool tall = p.OH >= 128 && (tiles8 >= slots || cost8 <= cost4) && !(p.remote_out && tiles8 < 2 * slots);
        static const int force_rows = [] { const char* e = getenv("NK_TILED_ROWS"); return e ? atoi(e) : 0; }();   // tuning: 8 or 4
        if (force_rows == 8) tall = true;
        if (force_rows == 4) tall = false;
        if (tall) st = f32 ? nk_tiled_dispatch_f32_tma8(ctx, int(KH), int(KW), of, If, Kf, p, &img) : nk_tiled_dispatch_f64_tma8(ctx, int(KH), int(KW), od, Id, Kd, p, &img);
        if (st == -1) st = f32 ? nk_tiled_dispatch_f32_tma4(ctx, int(KH), int(KW), of, If, Kf, p, &img) : nk_tiled_dispatch_f64_tma4(ctx, int(KH), int(KW), od, Id, Kd, p, &img);
        if (st != -1) family = NK_CONV_TMA;
    }
    if (st == -1 && ctx->conv_path != NK_CONV_TMA)
        st = f32 ? nk_tiled_dispatch_f32_ldgsts(ctx, int(KH), int(KW), of, If, Kf, p, nullptr) : nk_tiled_dispatch_f64_ldgsts(ctx, int(KH), int(KW), od, Id, Kd, p, nullptr);
    if (st == -1) return NK_OK;   // window size not instantiated / does not fit: generic family
    if (st != NK_OK) return st;
    ctx->last_conv_path = family;
    *handled = true;
    return NK_OK;
}
