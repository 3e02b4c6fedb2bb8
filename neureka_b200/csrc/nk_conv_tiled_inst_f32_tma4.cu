// float instantiations of the tiled stencil kernel (tma4 loader, 4 output rows per thread) for the window sizes
// that occur in practice; any other window is served by the generic gather family.
#include "nk_conv_tiled.cuh"

#define NK_CASE(H, W) if (kh == H && kw == W) return nk_launch_tiled<float, H, W, 4, true>(ctx, out, I, K, p, img)

int nk_tiled_dispatch_f32_tma4(nk_ctx* ctx, int kh, int kw, float* out, const float* I, const float* K, TiledPlan& p, const TmaImage* img) {
    NK_CASE(1, 1); NK_CASE(1, 2); NK_CASE(1, 3); NK_CASE(1, 4); NK_CASE(1, 5); NK_CASE(1, 7); NK_CASE(1, 9);
    NK_CASE(2, 2); NK_CASE(3, 3); NK_CASE(3, 5); NK_CASE(5, 3); NK_CASE(5, 5); NK_CASE(7, 7);
    return -1;
}
