// placeholder until the tiled family lands
#include "nk_conv_plan.h"
int nk_conv_tiled_try(nk_ctx*, int, nk_buf*, const NkView&, nk_buf*, const NkView&, nk_buf*, const NkView&, int, bool, bool* handled) {
    *handled = false;
    return NK_OK;
}
