// Routing of forward convolutions to the tiled stencil family: eligibility test, plan construction, tensor-map
// encoding and the (KH, KW) dispatch. The kernels themselves are instantiated per dtype / loader / rows-per-thread
// in nk_conv_tiled_inst_*.cu.

#include "nk_conv_tiled.cuh"

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

// Returns NK_OK with *handled = true when the call was launched on a tiled family, NK_OK with *handled = false
// when the views do not qualify (the caller then uses the generic family).
int nk_conv_tiled_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                      nk_buf* s2, const NkView& v2, int d, bool force, bool* handled) {
    *handled = false;
    if (d >= 0) return NK_OK;
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
        // 8 output rows per thread halve the shared-memory reads per multiply-add; worth it once the tile is filled
        // ... i.e. when the 64-row tiles alone give every SM several CTAs; small problems keep the 32-row tiles
        const int64_t tiles8 = int64_t((p.OW + 127) / 128) * ((p.OH + 63) / 64) * p.NP;
        const bool tall = p.OH >= 128 && tiles8 >= int64_t(ctx->prop.multiProcessorCount) * 4;
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
