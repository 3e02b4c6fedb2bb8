"""nk_sum_static, the allocation-free sum for hosts that own all of the GPU's memory themselves: it must return
exactly what nk_sum returns (same tiles, same order of additions), call after call, although all calls share one
fixed scratch array that still holds the previous call's partial sums; and it must refuse views whose partial sums
would not fit that array. This file is collected last on purpose: a run that stops at the first failure has then
already exercised everything else."""
import ctypes as C

import numpy as np
import pytest

from helpers import DevArray, cfgp
from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND

pytestmark = pytest.mark.gpu


def _sum_with(fn, device, src: DevArray, conf, out: DevArray, index: int):
    k, p = cfgp(conf)
    L.check(fn(device.ctx, src.nk_dtype, len(k) // 5, src.buf, p, out.buf, index), device.ctx)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_static_sum_equals_the_allocating_sum_on_consecutive_calls(device, dt):
    rng = np.random.default_rng(2024)
    # two calls in a row with different sizes: the second one finds the first one's partial sums in the array
    cases = [ND.of_shape([1_000_003]), ND.of_shape([37, 129]), ND.of_shape([300, 500]).sliced([150, 250], [3, 7], [2, 2]),
             ND.of_shape([5]), ND.of_shape([128 * 128 + 1])]
    for round_ in range(2):
        for conf in cases:
            n_data = conf.required_elements()
            src = DevArray(device, rng.standard_normal(n_data).astype(dt))
            out = DevArray(device, np.zeros(4, dtype=dt))
            _sum_with(L.lib.nk_sum, device, src, conf, out, 0)
            _sum_with(L.lib.nk_sum_static, device, src, conf, out, 1)
            _sum_with(L.lib.nk_sum_static, device, src, conf, out, 2)
            got = out.read()
            assert got[0] == got[1] == got[2], (conf.shape, got)
            assert got[3] == 0
            src.free(); out.free()


def test_static_sum_rejects_views_beyond_its_fixed_scratch(device):
    n = 34_000_000   # F32: ceil(n/128) + ceil(n/128^2) + 2 = 267,703 partial sums, the 1 MiB array holds 262,144
    buf = C.c_void_p()
    L.check(L.lib.nk_alloc(device.ctx, L.NK_F32, n, C.byref(buf)), device.ctx)
    out = DevArray(device, np.zeros(1, dtype=np.float32))
    try:
        k, p = cfgp(ND.of_shape([n]))
        st = L.lib.nk_sum_static(device.ctx, L.NK_F32, 1, buf, p, out.buf, 0)
        assert st == L.NK_ERR_UNSUPPORTED
        msg = L.lib.nk_last_error(device.ctx).decode()
        assert "fixed scratch array" in msg and "nk_sum" in msg
        # the allocating entry point takes the same view
        L.check(L.lib.nk_fill(device.ctx, buf, 0.5, 0, n), device.ctx)
        L.check(L.lib.nk_sum(device.ctx, L.NK_F32, 1, buf, p, out.buf, 0), device.ctx)
        assert out.read()[0] == pytest.approx(0.5 * n, rel=1e-3)
        with pytest.raises(ValueError):   # an integer dtype is refused (while the handles are still alive)
            L.check(L.lib.nk_sum_static(device.ctx, L.NK_I32, 1, out.buf, p, out.buf, 0), device.ctx)
    finally:
        L.lib.nk_free(device.ctx, buf)
        out.free()
