"""Side measurements of the other BASELINE configurations on one GPU (reported under "extra" by bench.py; the
headline line stays config 5). Everything goes through the C ABI with device-resident buffers and is timed with
the context's CUDA events after warm-up launches.

  cfg1  F32 [256,256] x [5,5]                  -> latency of one launch (the problem lives in L2: latency-bound)
  cfg2  F32 [64,512,512] x [64,3,3]            -> GB/s of algorithmic bytes, inputs rotated over 4 copies (> L2 in total)
  cfg3  F32 tanh(a*b+b), a [n,1,1024], b [1,m,1024] at n*m*1024 = 2^31 outputs (the full 2^33 does not exist in the
        reference: Java int sizes) -> GB/s of each of the three kernels the reference runs, plus the two gradient reductions
  cfg4  F64 [128,128,128] x [7,7,7] forward + gradient w.r.t. volume + gradient w.r.t. kernel -> GFLOP/s each
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .ndconf import NDConfiguration as ND


class _Buf:
    def __init__(self, dev, dtype, n, host=None):
        self.dev, self.n = dev, int(n)
        self.dt = L.NK_F32 if np.dtype(dtype) == np.float32 else L.NK_F64
        self.buf = C.c_void_p()
        L.check(L.lib.nk_alloc(dev.ctx, self.dt, self.n, C.byref(self.buf)), dev.ctx)
        if host is not None:
            h = np.ascontiguousarray(host, dtype=dtype)
            L.check(L.lib.nk_write(dev.ctx, self.buf, h.ctypes.data_as(C.c_void_p), 0, 0, h.size), dev.ctx)

    def free(self):
        if self.buf:
            L.lib.nk_free(self.dev.ctx, self.buf)
            self.buf = None


def _cfg(shape_or_conf):
    c = shape_or_conf if isinstance(shape_or_conf, ND) else ND.of_shape(shape_or_conf)
    a = c.as_inline_array()
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def _time(dev, fn, warm=3, reps=10):
    for _ in range(warm):
        fn(0)
    dev.sync()
    L.check(L.lib.nk_timer_begin(dev.ctx), dev.ctx)
    for i in range(reps):
        fn(i)
    ms = C.c_float(0)
    L.check(L.lib.nk_timer_end(dev.ctx, C.byref(ms)), dev.ctx)
    return float(ms.value) / reps


def _rand(dtype, n, dist, seed, p0, p1):
    a = np.zeros(n, dtype=dtype)
    dt = L.NK_F32 if np.dtype(dtype) == np.float32 else L.NK_F64
    L.lib.nk_jrand_fill(dt, dist, seed, p0, p1, a.ctypes.data_as(C.c_void_p), n)
    return a


def run_extra(dev, hbm_peak_gbs: float) -> dict:
    out = {}
    ctx = dev.ctx
    # measured FMA ceilings (register-resident loop): denominators for the FMA-bound kernels
    peaks = {}
    for name, dt in (("fp32", L.NK_F32), ("fp64", L.NK_F64)):
        v = C.c_double(0)
        L.check(L.lib.nk_measure_fma_peak(ctx, dt, C.byref(v)), ctx)
        peaks[name] = v.value
    out["measured_fma_peak_tflops"] = peaks

    # ---- cfg1 -----------------------------------------------------------------------------------------------------
    a = _Buf(dev, np.float32, 256 * 256, _rand(np.float32, 256 * 256, 0, 42, -1.0, 1.0))
    k = _Buf(dev, np.float32, 25, _rand(np.float32, 25, 0, 43, -1.0, 1.0))
    o = _Buf(dev, np.float32, 252 * 252)
    ca, pa = _cfg([256, 256]); ck, pk = _cfg([5, 5]); co, po = _cfg([252, 252])
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 2, o.buf, po, a.buf, pa, k.buf, pk, -1), ctx), 5, 200)
    out["cfg1_conv2d_256x256_k5"] = {"us_per_launch": ms * 1e3, "gflops": 3175200 / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel(),
                                     "note": "0.5 MB problem, L2 resident: launch-latency bound"}
    for b in (a, k, o): b.free()

    # ---- cfg2 -----------------------------------------------------------------------------------------------------
    n_in = 64 * 512 * 512
    host = _rand(np.float32, n_in, 1, 7, 0.0, 1.0)
    copies = [_Buf(dev, np.float32, n_in, host) for _ in range(4)]
    k = _Buf(dev, np.float32, 64 * 9, _rand(np.float32, 64 * 9, 1, 8, 0.0, 1.0))
    o = _Buf(dev, np.float32, 510 * 510)
    ca, pa = _cfg([64, 512, 512]); ck, pk = _cfg([64, 3, 3]); co, po = _cfg([1, 510, 510])
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 3, o.buf, po, copies[i % 4].buf, pa, k.buf, pk, -1), ctx), 4, 20)
    gbs = 68151568 / (ms * 1e-3) / 1e9
    out["cfg2_conv3d_64x512x512_k64x3x3"] = {"ms": ms, "gflops": 299635200 / (ms * 1e-3) / 1e9, "gbs": gbs, "frac_of_hbm_peak": gbs / hbm_peak_gbs,
                                             "kernel": dev.last_kernel(), "note": "4 rotating input copies (256 MiB) so that L2 cannot serve the reads"}
    for b in copies + [k, o]: b.free()

    # ---- cfg3 (scaled to 2^31 outputs) ---------------------------------------------------------------------------------
    n, m, kk = 2048, 1024, 1024
    a = _Buf(dev, np.float32, n * kk, _rand(np.float32, n * kk, 0, 3, -2.0, 2.0))
    b = _Buf(dev, np.float32, m * kk, _rand(np.float32, m * kk, 0, 4, -2.0, 2.0))
    N = n * m * kk
    t1, t2, y = (_Buf(dev, np.float32, N) for _ in range(3))
    ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
    r = {}
    ms = _time(dev, lambda i: L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t1.buf, po, a.buf, pa, b.buf, pb, -1), ctx), 2, 5)
    r["mul_broadcast"] = {"ms": ms, "gbs": (4.0 * (N + n * kk + m * kk)) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, t2.buf, po, t1.buf, po, b.buf, pb, -1), ctx), 2, 5)
    r["add_broadcast"] = {"ms": ms, "gbs": (4.0 * (2 * N + m * kk)) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, y.buf, po, t2.buf, po, -1), ctx), 2, 5)
    r["tanh"] = {"ms": ms, "gbs": (8.0 * N) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, t1.buf, po, t2.buf, po, 0), ctx), 2, 5)
    r["tanh_derivative"] = {"ms": ms, "gbs": (8.0 * N) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ga, gb = _Buf(dev, np.float32, n * kk), _Buf(dev, np.float32, m * kk)
    ms = _time(dev, lambda i: L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga.buf, pa, b.buf, pb, t1.buf, po, 0), ctx), 1, 3)
    r["grad_a_reduce"] = {"ms": ms, "gbs": (4.0 * (N + n * kk + m * kk)) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, gb.buf, pb, a.buf, pa, t1.buf, po, 0), ctx), 1, 3)
    r["grad_b_reduce"] = {"ms": ms, "gbs": (4.0 * (N + n * kk + m * kk)) / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    for v in r.values():
        v["frac_of_hbm_peak"] = v["gbs"] / hbm_peak_gbs
    r["tanh"]["note"] = ("F32 tanh is defined by the reference as a double-precision formula (exp + two divisions, ~22 FP64 "
                         "operations per element): the kernel is bound by the FP64 pipe, not by HBM")
    out["cfg3_broadcast_tanh_2048x1024x1024"] = r
    for bb in (a, b, t1, t2, y, ga, gb): bb.free()

    # ---- cfg3 forward as ONE run-time compiled kernel (no 32 GiB intermediates) -------------------------------------------
    try:
        r = {}
        h = C.c_void_p()
        L.check(L.lib.nk_fused_compile(ctx, L.NK_F32, 2, b"f_tanh(op_add(op_mul(x0,x1),x1))", C.byref(h)), ctx)
        h2 = C.c_void_p()
        L.check(L.lib.nk_fused_compile(ctx, L.NK_F32, 2, b"op_add(op_mul(x0,x1),x1)", C.byref(h2)), ctx)
        for name, (n, m, kk) in (("2048x1024x1024", (2048, 1024, 1024)), ("4096x2048x1024_full_size", (4096, 2048, 1024))):
            N = n * m * kk
            if dev.props.total_mem_bytes < N * 4 + (8 << 30):
                continue
            a = _Buf(dev, np.float32, n * kk, _rand(np.float32, n * kk, 0, 3, -2.0, 2.0))
            b = _Buf(dev, np.float32, m * kk, _rand(np.float32, m * kk, 0, 4, -2.0, 2.0))
            y = _Buf(dev, np.float32, N)
            ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
            bufs = (C.c_void_p * 2)(a.buf, b.buf)
            cfgs = (C.POINTER(C.c_int32) * 2)(pa, pb)
            nbytes = 4.0 * (N + n * kk + m * kk)
            ms = _time(dev, lambda i: L.check(L.lib.nk_fused_run(ctx, h, 3, y.buf, po, bufs, cfgs), ctx), 1, 3)
            ms2 = _time(dev, lambda i: L.check(L.lib.nk_fused_run(ctx, h2, 3, y.buf, po, bufs, cfgs), ctx), 1, 3)
            r[name] = {"tanh_affine_ms": ms, "tanh_affine_gbs": nbytes / (ms * 1e-3) / 1e9, "tanh_affine_frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs,
                       "affine_only_ms": ms2, "affine_only_gbs": nbytes / (ms2 * 1e-3) / 1e9, "affine_only_frac_of_hbm_peak": nbytes / (ms2 * 1e-3) / 1e9 / hbm_peak_gbs,
                       "kernel": dev.last_kernel()}
            for bb in (a, b, y): bb.free()
        r["note"] = ("tanh(i0*i1+i1) / i0*i1+i1 in one pass: 24 MiB read, the result written once; the tanh version is bound by the "
                     "FP64 pipe like the stand-alone tanh kernel, the affine version shows the kernel's own memory rate")
        L.lib.nk_fused_free(h); L.lib.nk_fused_free(h2)
        out["cfg3_fused_forward"] = r
    except Exception as e:
        out["cfg3_fused_forward"] = {"error": repr(e)}

    # ---- cfg3 at its full size: 2^33 outputs, op by op in the reference's order ------------------------------------------
    # 4096*2048*1024 elements overflow Java's int sizes, so the reference itself cannot hold this tensor; here every
    # intermediate is one 32 GiB buffer (64-bit offsets throughout). Needs ~100 GiB free.
    try:
        if dev.props.total_mem_bytes >= 150 * (1 << 30):
            n, m, kk = 4096, 2048, 1024
            N = n * m * kk
            a = _Buf(dev, np.float32, n * kk, _rand(np.float32, n * kk, 0, 3, -2.0, 2.0))
            b = _Buf(dev, np.float32, m * kk, _rand(np.float32, m * kk, 0, 4, -2.0, 2.0))
            t2, y, g = (_Buf(dev, np.float32, N) for _ in range(3))
            ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
            ga, gb = _Buf(dev, np.float32, n * kk), _Buf(dev, np.float32, m * kk)
            steps = [
                ("mul_broadcast", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t2.buf, po, a.buf, pa, b.buf, pb, -1), 4.0 * (N + n * kk + m * kk)),
                ("add_broadcast_in_place", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, y.buf, po, t2.buf, po, b.buf, pb, -1), 4.0 * (2 * N + m * kk)),
                ("tanh", lambda i: L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g.buf, po, y.buf, po, -1), 8.0 * N),
                ("tanh_derivative", lambda i: L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g.buf, po, y.buf, po, 0), 8.0 * N),
                ("grad_a_reduce", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga.buf, pa, b.buf, pb, g.buf, po, 0), 4.0 * (N + n * kk + m * kk)),
                ("grad_b_reduce_mul", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, gb.buf, pb, a.buf, pa, g.buf, po, 0), 4.0 * (N + n * kk + m * kk)),
            ]
            r = {}
            total_ms = 0.0
            for name, fn, nbytes in steps:
                ms = _time(dev, lambda i, fn=fn: L.check(fn(i), ctx), 1, 2)
                total_ms += ms
                r[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel()}
            r["forward_plus_backward_ms"] = total_ms
            r["note"] = "2^33 F32 outputs per intermediate (32 GiB each); beyond the reference's int-sized tensors"
            out["cfg3_full_size_4096x2048x1024"] = r
            for bb in (a, b, t2, y, g, ga, gb): bb.free()
    except Exception as e:   # a side measurement must not take the others down
        out["cfg3_full_size_4096x2048x1024"] = {"error": repr(e)}

    # ---- contraction-shaped `x` (Tensor.convDot: [M,K,1] x [1,K,N]) ------------------------------------------------------
    try:
        r = {}
        for name, dt, npdt, n, fma_peak in (("f32_4096", L.NK_F32, np.float32, 4096, "fp32"), ("f64_2048", L.NK_F64, np.float64, 2048, "fp64"),
                                            ("f32_1024", L.NK_F32, np.float32, 1024, "fp32")):
            rng = np.random.default_rng(5)
            A = _Buf(dev, npdt, n * n, rng.standard_normal(n * n).astype(npdt))
            B = _Buf(dev, npdt, n * n, rng.standard_normal(n * n).astype(npdt))
            O = _Buf(dev, npdt, n * n)
            c1, p1 = _cfg([n, n, 1]); c2, p2 = _cfg([1, n, n]); c0, p0 = _cfg([n, 1, n])
            flops = 2.0 * n * n * n
            ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, dt, 3, O.buf, p0, A.buf, p1, B.buf, p2, -1), ctx), 2, 5)
            r[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "kernel": dev.last_kernel(),
                       "frac_of_measured_fma_peak": flops / (ms * 1e-3) / 1e12 / out["measured_fma_peak_tflops"][fma_peak]}
            if n == 1024:   # the gather family on the same call, for scale
                dev.set_conv_path(L.NK_CONV_GENERIC)
                ms_g = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, dt, 3, O.buf, p0, A.buf, p1, B.buf, p2, -1), ctx), 1, 3)
                dev.set_conv_path(L.NK_CONV_AUTO)
                r[name]["gather_family_ms"] = ms_g
            for bb in (A, B, O): bb.free()
        out["contraction_MxKx1_x_1xKxN"] = r
    except Exception as e:
        out["contraction_MxKx1_x_1xKxN"] = {"error": repr(e)}

    # ---- cfg5's forward pass on the slabs a rank holds at 4 and 8 GPUs (what bounds the multi-GPU rows) ---------------------
    try:
        r = {}
        for name, rows in (("one_of_8_ranks_260_rows", 260), ("one_of_4_ranks_515_rows", 515)):
            Bn, Cn, W, KH = 8, 32, 2048, 5
            img = _Buf(dev, np.float32, Bn * Cn * rows * W)
            L.check(L.lib.nk_fill(ctx, img.buf, C.c_double(0.5), 0, Bn * Cn * rows * W), ctx)
            ker = _Buf(dev, np.float32, Cn * KH * KH, _rand(np.float32, Cn * KH * KH, 1, 6, 0.0, 0.2))
            o = _Buf(dev, np.float32, Bn * (rows - 4) * (W - 4))
            ci, pi_ = _cfg([Bn, Cn, rows, W]); ckk, pkk = _cfg([1, Cn, KH, KH]); co_, po_ = _cfg([Bn, 1, rows - 4, W - 4])
            ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, o.buf, po_, img.buf, pi_, ker.buf, pkk, -1), ctx), 3, 20)
            flops = 2.0 * Bn * (rows - 4) * (W - 4) * Cn * KH * KH
            r[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "kernel": dev.last_kernel()}
            for bb in (img, ker, o): bb.free()
        out["cfg5_forward_on_one_rank_slab"] = r
    except Exception as e:
        out["cfg5_forward_on_one_rank_slab"] = {"error": repr(e)}

    # ---- gradients of cfg5's convolution (error seeded, uniform [-1,1]) ---------------------------------------------------
    try:
        Bn, Cn, H, W, KH = 8, 32, 2048, 2048, 5
        OH, OW = H - KH + 1, W - KH + 1
        img = _Buf(dev, np.float32, Bn * Cn * H * W)
        L.check(L.lib.nk_fill(ctx, img.buf, C.c_double(0.5), 0, Bn * Cn * H * W), ctx)
        err = _Buf(dev, np.float32, Bn * OH * OW, _rand(np.float32, Bn * OH * OW, 0, 9, -1.0, 1.0))
        ker = _Buf(dev, np.float32, Cn * KH * KH, _rand(np.float32, Cn * KH * KH, 1, 6, 0.0, 0.2))
        gimg, gker = _Buf(dev, np.float32, Bn * Cn * H * W), _Buf(dev, np.float32, Cn * KH * KH)
        ci, pi_ = _cfg([Bn, Cn, H, W]); ce, pe = _cfg([Bn, 1, OH, OW]); ckk, pkk = _cfg([1, Cn, KH, KH])
        flops = 2.0 * Bn * OH * OW * Cn * KH * KH
        r = {}
        ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gimg.buf, pi_, ker.buf, pkk, err.buf, pe, 0), ctx), 2, 5)
        nbytes = 4.0 * (Bn * Cn * H * W + Bn * OH * OW + Cn * KH * KH)
        r["grad_image"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9,
                           "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel(),
                           "note": "write-bound: 4.29 GB of gradient written, 0.13 GB of error read"}
        ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gker.buf, pkk, img.buf, pi_, err.buf, pe, 0), ctx), 2, 5)
        r["grad_kernel"] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "gbs": nbytes / (ms * 1e-3) / 1e9,
                            "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel()}
        out["cfg5_gradients"] = r
        for bb in (img, err, ker, gimg, gker): bb.free()
    except Exception as e:
        out["cfg5_gradients"] = {"error": repr(e)}

    # ---- cfg4 -----------------------------------------------------------------------------------------------------
    v = _Buf(dev, np.float64, 128 ** 3, _rand(np.float64, 128 ** 3, 1, 11, 0.0, 1.0))
    k = _Buf(dev, np.float64, 343, _rand(np.float64, 343, 1, 12, 0.0, 0.1))
    yb = _Buf(dev, np.float64, 122 ** 3)
    gv, gk = _Buf(dev, np.float64, 128 ** 3), _Buf(dev, np.float64, 343)
    cv, pv = _cfg([128] * 3); ck, pk = _cfg([7] * 3); cy, py = _cfg([122] * 3)
    flops = 1245671728.0
    r = {}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, yb.buf, py, v.buf, pv, k.buf, pk, -1), ctx), 3, 10)
    r["forward"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    # gradients for error = y itself (any error tensor does): XConvRight(error, other, zeros) -> (drain, other, error), d = 0
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, gv.buf, pv, k.buf, pk, yb.buf, py, 0), ctx), 2, 5)
    r["grad_volume"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, gk.buf, pk, v.buf, pv, yb.buf, py, 0), ctx), 2, 5)
    r["grad_kernel"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    for v_ in r.values():
        v_["frac_of_fp64_fma_peak"] = v_["gflops"] / 1e3 / peaks["fp64"]
    out["cfg4_conv3d_f64_128_k7"] = r
    for bb in (v, k, yb, gv, gk): bb.free()
    return out


def run_small_broadcast(dev, hbm_peak_gbs: float) -> dict:
    """The broadcast / elementwise / reduction kernels of config 3 on a case small enough for a multi-pass profiler
    capture and still far larger than L2: a [1024,1,1024], b [1,512,1024] -> 2^29 outputs (2 GiB per tensor)."""
    ctx = dev.ctx
    n, m, kk = 1024, 512, 1024
    N = n * m * kk
    a = _Buf(dev, np.float32, n * kk, _rand(np.float32, n * kk, 0, 3, -2.0, 2.0))
    b = _Buf(dev, np.float32, m * kk, _rand(np.float32, m * kk, 0, 4, -2.0, 2.0))
    t1, t2 = _Buf(dev, np.float32, N), _Buf(dev, np.float32, N)
    ga = _Buf(dev, np.float32, n * kk)
    ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
    out = {}
    for name, fn, nbytes in (
            ("mul_broadcast", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t1.buf, po, a.buf, pa, b.buf, pb, -1), 4.0 * (N + n * kk + m * kk)),
            ("add_broadcast", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, t2.buf, po, t1.buf, po, b.buf, pb, -1), 4.0 * (2 * N + m * kk)),
            ("relu", lambda i: L.lib.nk_unary(ctx, L.FUN["relu"], L.NK_F32, 3, t1.buf, po, t2.buf, po, -1), 8.0 * N),
            ("grad_a_reduce", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga.buf, pa, b.buf, pb, t1.buf, po, 0), 4.0 * (N + n * kk + m * kk))):
        ms = _time(dev, lambda i, fn=fn: L.check(fn(i), ctx), 2, 4)
        out[name] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel()}
    for bb in (a, b, t1, t2, ga): bb.free()
    return out


def run_small_gradients(dev, hbm_peak_gbs: float) -> dict:
    """Both gradients of an [8,32,512,2048] x [1,32,5,5] convolution (1 GiB image): the profiler-sized case of the
    config 5 gradient kernels."""
    ctx = dev.ctx
    Bn, Cn, H, W, KH = 8, 32, 512, 2048, 5
    OH, OW = H - KH + 1, W - KH + 1
    img = _Buf(dev, np.float32, Bn * Cn * H * W)
    L.check(L.lib.nk_fill(ctx, img.buf, C.c_double(0.5), 0, Bn * Cn * H * W), ctx)
    err = _Buf(dev, np.float32, Bn * OH * OW, _rand(np.float32, Bn * OH * OW, 0, 9, -1.0, 1.0))
    ker = _Buf(dev, np.float32, Cn * KH * KH, _rand(np.float32, Cn * KH * KH, 1, 6, 0.0, 0.2))
    gimg, gker = _Buf(dev, np.float32, Bn * Cn * H * W), _Buf(dev, np.float32, Cn * KH * KH)
    ci, pi_ = _cfg([Bn, Cn, H, W]); ce, pe = _cfg([Bn, 1, OH, OW]); ckk, pkk = _cfg([1, Cn, KH, KH])
    nbytes = 4.0 * (Bn * Cn * H * W + Bn * OH * OW + Cn * KH * KH)
    out = {}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gimg.buf, pi_, ker.buf, pkk, err.buf, pe, 0), ctx), 2, 4)
    out["grad_image"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gker.buf, pkk, img.buf, pi_, err.buf, pe, 0), ctx), 2, 4)
    out["grad_kernel"] = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm_peak_gbs, "kernel": dev.last_kernel()}
    for bb in (img, err, ker, gimg, gker): bb.free()
    return out


def run_small_contraction(dev) -> dict:
    """[4096,4096,1] x [1,4096,4096] in F32 alone (201 MB of operands and result): the command a profiler is pointed at."""
    ctx = dev.ctx
    n = 4096
    rng = np.random.default_rng(5)
    A = _Buf(dev, np.float32, n * n, rng.standard_normal(n * n).astype(np.float32))
    B = _Buf(dev, np.float32, n * n, rng.standard_normal(n * n).astype(np.float32))
    O = _Buf(dev, np.float32, n * n)
    c1, p1 = _cfg([n, n, 1]); c2, p2 = _cfg([1, n, n]); c0, p0 = _cfg([n, 1, n])
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 3, O.buf, p0, A.buf, p1, B.buf, p2, -1), ctx), 2, 4)
    out = {"ms": ms, "tflops": 2.0 * n * n * n / (ms * 1e-3) / 1e12, "kernel": dev.last_kernel()}
    for bb in (A, B, O): bb.free()
    return out


if __name__ == "__main__":
    # python -m neureka_b200.extra_bench : the side measurements alone, as JSON (also the command ncu is pointed at);
    # --small-broadcast : only a 2 GiB case of the broadcast / elementwise / reduction kernels (for full-set captures)
    # --small-contraction : only the 4096^3 F32 contraction
    # --small-gradients : only the two gradients of a quarter-height config 5 convolution
    import json
    import os
    import sys
    from .device import CudaDevice
    peak = 6558.7
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak = float(json.load(f)["hbm_gbs"])
    if "--small-gradients" in sys.argv[1:]:
        print(json.dumps(run_small_gradients(CudaDevice.get(0), peak), indent=1))
    elif "--small-contraction" in sys.argv[1:]:
        print(json.dumps(run_small_contraction(CudaDevice.get(0)), indent=1))
    elif "--small-broadcast" in sys.argv[1:]:
        print(json.dumps(run_small_broadcast(CudaDevice.get(0), peak), indent=1))
    else:
        print(json.dumps(run_extra(CudaDevice.get(0), peak), indent=1))
