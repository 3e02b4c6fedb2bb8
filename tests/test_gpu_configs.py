"""The BASELINE configurations themselves, on their seeded inputs (java.util.Random-compatible streams), against the
CPU oracle: full output where the oracle finishes in seconds, otherwise oracle spot checks on sampled output ranges
plus size-independent properties (linearity in the kernel, shift equivariance, gradient = adjoint identity).

Every comparison of a convolution result uses the stated tolerance per element with no extra factor:
|gpu - oracle| <= 1e-5 (F32) / 1e-12 (F64) x sum|a||b| (helpers.assert_conv_close)."""
import ctypes as C

import numpy as np
import pytest

import baseline_configs as BC
from helpers import DevArray, assert_conv_close, cfgp, gpu_conv
from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND

pytestmark = pytest.mark.gpu


def test_config1_conv2d_matches_the_simple_cpu_convolution(device, oracle):
    a, k = BC.cfg1_inputs()   # one stream of seed 42: the image, then the kernel
    co, ca, ck = ND.of_shape([252, 252]), ND.of_shape([256, 256]), ND.of_shape([5, 5])
    ref = np.zeros(co.size, dtype=np.float32)
    assert oracle.conv(ref, co.as_inline_array(), a, ca.as_inline_array(), k, ck.as_inline_array()) == 1   # SimpleCPUConvolution path
    scale = np.zeros(co.size, dtype=np.float32)
    oracle.conv(scale, co.as_inline_array(), np.abs(a), ca.as_inline_array(), np.abs(k), ck.as_inline_array())
    got = gpu_conv(device, np.zeros(co.size, dtype=np.float32), co, a, ca, k, ck)
    assert_conv_close(got, ref, scale, "config 1")
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()


def test_config2_channel_collapsing_conv(device, oracle):
    a, k = BC.cfg2_inputs()   # one N(0,1) stream of seed 7: the image, then the kernel
    co, ca, ck = ND.of_shape([1, 510, 510]), ND.of_shape([64, 512, 512]), ND.of_shape([64, 3, 3])
    ref = np.zeros(co.size, dtype=np.float32)
    assert oracle.conv(ref, co.as_inline_array(), a, ca.as_inline_array(), k, ck.as_inline_array(), threads=8) == 0   # general nd path
    scale = np.zeros(co.size, dtype=np.float32)
    oracle.conv(scale, co.as_inline_array(), np.abs(a), ca.as_inline_array(), np.abs(k), ck.as_inline_array(), threads=8)
    got = gpu_conv(device, np.zeros(co.size, dtype=np.float32), co, a, ca, k, ck)
    assert_conv_close(got, ref, scale, "config 2")
    assert np.abs(got - ref).max() <= 1e-5 * np.abs(ref).max()


def test_config4_f64_forward_and_both_gradients(device, oracle):
    v, k = BC.cfg4_inputs()
    cv, ck, cy = ND.of_shape([128] * 3), ND.of_shape([7] * 3), ND.of_shape([122] * 3)
    iv, ik, iy = cv.as_inline_array(), ck.as_inline_array(), cy.as_inline_array()
    av, ak = np.abs(v), np.abs(k)
    y = gpu_conv(device, np.zeros(cy.size), cy, v, cv, k, ck)
    # forward: oracle on sampled ranges of the output (the full state machine would take minutes)
    rng = np.random.default_rng(4)
    ref, scale = np.zeros(cy.size), np.zeros(cy.size)
    for s in [0, cy.size - 3000] + [int(x) for x in rng.integers(0, cy.size - 3000, size=6)]:
        oracle.conv_range(ref, iy, v, iv, k, ik, -1, s, s + 3000)
        oracle.conv_range(scale, iy, av, iv, ak, ik, -1, s, s + 3000)
        seg = slice(s, s + 3000)
        assert_conv_close(y[seg], ref[seg], scale[seg], f"config 4 forward, range at {s}")
    # backward of sum(y): error = ones
    err = np.ones(cy.size)
    gk = gpu_conv(device, np.zeros(343), ck, v, cv, err, cy, d=0)             # (drain = kernel-shaped, t1 = volume, t2 = error)
    gv = gpu_conv(device, np.zeros(128 ** 3), cv, k, ck, err, cy, d=0)         # (drain = volume-shaped, t1 = kernel, t2 = error)
    # grad wrt kernel with error = ones is a box sum of the volume: all 343 taps against summed-area tables in
    # extended precision, bound 1e-12 x the box sum of |v|
    def boxes(vol):
        csum = np.zeros((129, 129, 129), dtype=np.longdouble)
        csum[1:, 1:, 1:] = vol.reshape(128, 128, 128).astype(np.longdouble).cumsum(0).cumsum(1).cumsum(2)
        out = []
        for z in range(7):
            for yy in range(7):
                for x in range(7):
                    z1, y1, x1 = z + 122, yy + 122, x + 122
                    out.append(csum[z1, y1, x1] - csum[z, y1, x1] - csum[z1, yy, x1] - csum[z1, y1, x] + csum[z, yy, x1]
                               + csum[z, y1, x] + csum[z1, yy, x] - csum[z, yy, x])
        return np.array(out, dtype=np.longdouble)
    want_gk, scale_gk = boxes(v), boxes(av)
    assert np.all(np.abs(gk - want_gk) <= 1e-12 * scale_gk), float(np.max(np.abs(gk - want_gk) / scale_gk))
    # the oracle's general deconvolution on two taps (122^3 terms each), same bound
    ref_gk = np.zeros(343)
    oracle.conv_range(ref_gk, ik, v, iv, err, iy, 0, 170, 172)
    assert_conv_close(gk[170:172], ref_gk[170:172], np.asarray(scale_gk[170:172], dtype=np.float64), "config 4 kernel gradient")
    # grad wrt volume: oracle on sampled ranges (each element visits all of the error in the reference: keep it short)
    ref_gv, scale_gv = np.zeros(128 ** 3), np.zeros(128 ** 3)
    for s in (0, 128 * 128 * 64 + 128 * 60 + 50, 128 ** 3 - 2):
        oracle.conv_range(ref_gv, iv, k, ik, err, iy, 0, s, s + 2)
        oracle.conv_range(scale_gv, iv, ak, ik, err, iy, 0, s, s + 2)
        assert_conv_close(gv[s:s + 2], ref_gv[s:s + 2], scale_gv[s:s + 2], f"config 4 volume gradient at {s}")
    # error = ones: every volume gradient is a box sum of the kernel -- all 128^3 of them against the same tables idea
    kc = np.zeros((8, 8, 8), dtype=np.longdouble)
    kc[1:, 1:, 1:] = k.reshape(7, 7, 7).astype(np.longdouble).cumsum(0).cumsum(1).cumsum(2)
    ka = np.zeros((8, 8, 8), dtype=np.longdouble)
    ka[1:, 1:, 1:] = ak.reshape(7, 7, 7).astype(np.longdouble).cumsum(0).cumsum(1).cumsum(2)
    idx = np.arange(128)
    lo, hi = np.maximum(idx - 121, 0), np.minimum(idx, 6) + 1     # taps t with 0 <= p - t < 122
    def box3(c):
        L0, H0 = lo[:, None, None], hi[:, None, None]
        L1, H1 = lo[None, :, None], hi[None, :, None]
        L2, H2 = lo[None, None, :], hi[None, None, :]
        return (c[H0, H1, H2] - c[L0, H1, H2] - c[H0, L1, H2] - c[H0, H1, L2] + c[L0, L1, H2] + c[L0, H1, L2] + c[H0, L1, L2] - c[L0, L1, L2])
    want_gv, scale_all = box3(kc).reshape(-1), box3(ka).reshape(-1)
    assert np.all(np.abs(gv - want_gv) <= 1e-12 * scale_all)
    # adjoint identity <conv(v,k), e> = <v, grad_v(e)> = <k, grad_k(e)> for a random error
    e = rng.standard_normal(cy.size)
    gk_e = gpu_conv(device, np.zeros(343), ck, v, cv, e, cy, d=0)
    gv_e = gpu_conv(device, np.zeros(128 ** 3), cv, k, ck, e, cy, d=0)
    lhs = float(np.dot(y, e))
    assert float(np.dot(v, gv_e)) == pytest.approx(lhs, rel=1e-10)
    assert float(np.dot(k, gk_e)) == pytest.approx(lhs, rel=1e-10)


def test_config5_full_size_on_one_gpu(device, oracle):
    """4 GiB input: oracle spot checks on sampled output ranges, plus properties that hold at any size."""
    a_shape, k_shape, o_shape = [8, 32, 2048, 2048], [1, 32, 5, 5], [8, 1, 2044, 2044]
    n_in, n_out = int(np.prod(a_shape)), int(np.prod(o_shape))
    a = BC.cfg5_image()
    k = BC.cfg5_kernel()
    A = DevArray(device, a)
    K = DevArray(device, k)
    O = DevArray(device, np.zeros(1, dtype=np.float32))
    O.free()
    buf = C.c_void_p()
    L.check(L.lib.nk_alloc(device.ctx, L.NK_F32, n_out, C.byref(buf)), device.ctx)
    ka, pa = cfgp(ND.of_shape(a_shape)); kk, pk = cfgp(ND.of_shape(k_shape)); ko, po = cfgp(ND.of_shape(o_shape))
    L.check(L.lib.nk_conv(device.ctx, L.NK_F32, 4, buf, po, A.buf, pa, K.buf, pk, -1), device.ctx)
    y = np.empty(n_out, dtype=np.float32)
    L.check(L.lib.nk_read(device.ctx, buf, y.ctypes.data_as(C.c_void_p), 0, n_out), device.ctx)
    assert device.last_conv_path() in (L.NK_CONV_TILED, L.NK_CONV_TMA)
    rng = np.random.default_rng(55)
    ref = np.zeros(n_out, dtype=np.float32)
    starts = [0, n_out - 500, 2044 * 2044 * 3 + 2044 * 2043 + 1500] + [int(s) for s in rng.integers(0, n_out - 500, size=5)]
    scale = np.zeros(n_out, dtype=np.float32)
    ak = np.abs(k)    # the image is uniform on [0, 1): already non-negative
    for s in starts:
        oracle.conv_range(ref, ko, a, ka, k, kk, -1, s, s + 500)
        oracle.conv_range(scale, ko, a, ka, ak, kk, -1, s, s + 500)
        assert_conv_close(y[s:s + 500], ref[s:s + 500], scale[s:s + 500], f"config 5, range at {s}")
        assert np.abs(y[s:s + 500] - ref[s:s + 500]).max() <= 1e-5 * np.abs(ref[s:s + 500]).max()
    # linearity in the kernel: conv(a, 2k) == 2 conv(a, k) exactly (power-of-two scaling)
    K2 = DevArray(device, k * 2)
    L.check(L.lib.nk_conv(device.ctx, L.NK_F32, 4, buf, po, A.buf, pa, K2.buf, pk, -1), device.ctx)
    y2 = np.empty(n_out, dtype=np.float32)
    L.check(L.lib.nk_read(device.ctx, buf, y2.ctypes.data_as(C.c_void_p), 0, n_out), device.ctx)
    assert np.array_equal(y2, 2 * y)
    # a delta kernel copies a shifted window of one channel: exact
    delta = np.zeros(800, dtype=np.float32)
    delta[7 * 25 + 2 * 5 + 3] = 1.0     # channel 7, tap (2, 3)
    KD = DevArray(device, delta)
    L.check(L.lib.nk_conv(device.ctx, L.NK_F32, 4, buf, po, A.buf, pa, KD.buf, pk, -1), device.ctx)
    L.check(L.lib.nk_read(device.ctx, buf, y2.ctypes.data_as(C.c_void_p), 0, n_out), device.ctx)
    want = a.reshape(a_shape)[:, 7, 2:2 + 2044, 3:3 + 2044]
    assert np.array_equal(y2.reshape(8, 2044, 2044), want)
    L.lib.nk_free(device.ctx, buf)
    for b in (A, K, K2, KD):
        b.free()


def test_config3_full_size_beyond_java_int(device, oracle):
    """BASELINE config 3 at its real size: y = tanh(a*b + b) with a [4096,1,1024], b [1,2048,1024] -> 2^33 outputs
    (32 GiB per tensor, more elements than a Java int can count, so the reference cannot even allocate it). The three
    kernels run op by op like the reference would; sampled windows of the result are compared with the oracle's
    scalar functions (<= 1 ulp), and the reduced gradients of sum(y) with float64 sums over the sampled columns."""
    import ctypes as C
    if device.props.total_mem_bytes < 150 * (1 << 30):
        pytest.skip("needs ~100 GiB of device memory")
    n, m, k = 4096, 2048, 1024
    N = n * m * k
    a_h, b_h = BC.cfg3_inputs()   # one uniform stream of seed 3: a, then b
    A, B = DevArray(device, a_h), DevArray(device, b_h)
    bufs = []
    for _ in range(2):
        p = C.c_void_p()
        L.check(L.lib.nk_alloc(device.ctx, L.NK_F32, N, C.byref(p)), device.ctx)
        bufs.append(p)
    t, y = bufs
    ka, pa = cfgp(ND.of_shape([n, 1, k])); kb, pb = cfgp(ND.of_shape([1, m, k])); ko, po = cfgp(ND.of_shape([n, m, k]))
    ctx = device.ctx
    L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t, po, A.buf, pa, B.buf, pb, -1), ctx)
    L.check(L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, y, po, t, po, B.buf, pb, -1), ctx)      # y = a*b + b
    L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, t, po, y, po, -1), ctx)                    # t = tanh(y)
    rng = np.random.default_rng(33)
    a3, b3 = a_h.reshape(n, 1, k), b_h.reshape(1, m, k)
    win = 4096
    starts = [0, N - win, (1 << 32) - 100, (1 << 31) + 12345] + [int(s) for s in rng.integers(0, N - win, size=6)]
    for s0 in starts:
        got = np.empty(win, dtype=np.float32)
        L.check(L.lib.nk_read(ctx, t, got.ctypes.data_as(C.c_void_p), s0, win), ctx)
        idx = np.arange(s0, s0 + win, dtype=np.int64)
        i, j, kk = idx // (m * k), (idx // k) % m, idx % k
        u = (a_h[i * k + kk] * b_h[j * k + kk]).astype(np.float32) + b_h[j * k + kk]
        want = np.zeros(win, dtype=np.float32)
        cw = ND.of_shape([win]).as_inline_array()
        oracle.unary("tanh", want, cw, np.ascontiguousarray(u, dtype=np.float32), cw)
        d = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
        assert d.max() <= 1, (s0, d.max())
    # g = tanh'(y) in place of y's consumer buffer, then the reduced gradients of sum(tanh(...))
    L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, t, po, y, po, 0), ctx)
    GA, GB = DevArray(device, np.zeros(n * k, dtype=np.float32)), DevArray(device, np.zeros(m * k, dtype=np.float32))
    L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, GA.buf, pa, B.buf, pb, t, po, 0), ctx)   # da = sum_j g*b
    L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, GB.buf, pb, A.buf, pa, t, po, 0), ctx)   # sum_i g*a
    ga, gb = GA.read().reshape(n, k), GB.read().reshape(m, k)
    # reference values for a few (i, :) rows of da and (j, :) rows of db: need g over a whole line of the big tensor
    for i in (0, 1777, n - 1):
        row = np.empty(m * k, dtype=np.float32)
        L.check(L.lib.nk_read(ctx, t, row.ctypes.data_as(C.c_void_p), i * m * k, m * k), ctx)
        want = (row.reshape(m, k).astype(np.float64) * b_h.reshape(m, k)).sum(axis=0)
        np.testing.assert_allclose(ga[i], want, rtol=2e-5, atol=2e-4)
    for j in (0, 999, m - 1):
        col = np.empty((n, k), dtype=np.float32)
        # db[j, :] = sum_i g[i, j, :] * a[i, :]; read g[:, j, :] row by row (4096 reads of 4 KB)
        for i in range(n):
            L.check(L.lib.nk_read(ctx, t, col[i].ctypes.data_as(C.c_void_p), (i * m + j) * k, k), ctx)
        want = (col.astype(np.float64) * a_h.reshape(n, k)).sum(axis=0)
        np.testing.assert_allclose(gb[j], want, rtol=2e-5, atol=2e-4)
    for p in bufs:
        L.lib.nk_free(ctx, p)
    for x in (A, B, GA, GB):
        x.free()
