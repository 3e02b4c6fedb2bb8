// Routing of forward convolutions to the tiled stencil family: eligibility test, plan construction and the
// (KH, KW) dispatch. The kernels themselves are instantiated per dtype in nk_conv_tiled_f32.cu / _f64.cu.

#include "nk_conv_tiled.cuh"

int nk_tiled_dispatch_f32(nk_ctx* ctx, int kh, int kw, float* out, const float* I, const float* K, TiledPlan& p);
int nk_tiled_dispatch_f64(nk_ctx* ctx, int kh, int kw, double* out, const double* I, const double* K, TiledPlan& p);

namespace {

bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

}  // namespace

// Returns NK_OK with *handled = true when the call was launched on the tiled family, NK_OK with
// *handled = false when the views do not qualify (the caller then uses the generic family).
int nk_conv_tiled_try(nk_ctx* ctx, int dtype, nk_buf* drn, const NkView& v0, nk_buf* s1, const NkView& v1,
                      nk_buf* s2, const NkView& v2, int d, bool force, bool* handled) {
    *handled = false;
    if (d >= 0) return NK_OK;
    if (ctx->conv_path == NK_CONV_TMA) return NK_OK;   // no TMA variant in this build: report "does not apply"
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
    if (rank >= 2) {
        const int Y = rank - 2;
        const bool window_y = vi.shape[Y] >= vk.shape[Y] && vk.shape[Y] <= 7 && vi.shape[Y] > 1;
        if (window_y) {
            KH = vk.shape[Y]; IH = vi.shape[Y]; OH = IH - KH + 1;
            if (v0.shape[Y] != OH) return NK_OK;
            sIy = vi.estride[Y]; sKy = vk.estride[Y]; sOy = v0.estride[Y];
            n_outer = rank - 2;
        }
    }
    if (n_outer > NK_TILED_MAX_OUTER) return NK_OK;
    TiledPlan p;
    memset(&p, 0, sizeof(p));
    p.n_outer = n_outer;
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

    int st;
    if (dtype == NK_F32) st = nk_tiled_dispatch_f32(ctx, int(KH), int(KW), (float*)drn->ptr, (const float*)bi->ptr, (const float*)bk->ptr, p);
    else st = nk_tiled_dispatch_f64(ctx, int(KH), int(KW), (double*)drn->ptr, (const double*)bi->ptr, (const double*)bk->ptr, p);
    if (st == -1) return NK_OK;   // window size not instantiated / does not fit: generic family
    if (st != NK_OK) return st;
    ctx->last_conv_path = NK_CONV_TILED;
    *handled = true;
    return NK_OK;
}
