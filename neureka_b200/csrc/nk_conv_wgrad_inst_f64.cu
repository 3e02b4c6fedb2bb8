// double instantiations of the kernel-gradient reduction for the window sizes that occur in practice; any other
// window is served by the generic gather family.
#include "nk_conv_wgrad.cuh"

#define NK_CASE(H, W) if (kh == H && kw == W) return nk_launch_wgrad<double, H, W>(ctx, out, p, imgA, imgE)

int nk_wgrad_dispatch_f64(nk_ctx* ctx, int kh, int kw, double* out, WgradPlan& p, const TmaImage& imgA, const TmaImage& imgE) {
    NK_CASE(1, 1); NK_CASE(1, 3); NK_CASE(1, 5); NK_CASE(2, 2); NK_CASE(3, 3); NK_CASE(3, 5); NK_CASE(5, 3); NK_CASE(5, 5); NK_CASE(7, 7);
    return -1;
}
