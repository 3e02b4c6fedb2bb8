"""Side measurements of the other BASELINE configurations on one GPU (reported under "extra" by bench.py; the
headline line stays config 5).

    python bench_extra.py [--only SECTION[,SECTION...]] [--small]

prints them alone as JSON. --only runs the named sections (see SECTIONS); --small swaps a section's workload for one
of the same kernels that holds a few GB at most (still far larger than L2) -- the form a multi-pass profiler capture
needs. Everything goes through the C ABI with device-resident buffers and is timed with the context's CUDA events
after warm-up launches.

  cfg5_group  config 5 through the in-process device group on every visible GPU (only with --only cfg5_group)
  cfg1  F32 [256,256] x [5,5]                  -> latency of one launch (the problem lives in L2: latency-bound)
  cfg2  F32 [64,512,512] x [64,3,3]            -> GB/s of algorithmic bytes, inputs rotated over 4 copies (> L2 in total)
  cfg3  F32 tanh(a*b+b), a [n,1,1024], b [1,m,1024] at n*m*1024 = 2^31 outputs and at the full 2^33 (which cannot exist
        in the reference: Java int sizes) -> GB/s of each kernel the reference runs, the gradient reductions, and the
        run-time compiled fused forms
  cfg4  F64 [128,128,128] x [7,7,7] forward + gradient w.r.t. volume + gradient w.r.t. kernel -> GFLOP/s each
  cfg5  the slabs one rank holds at 4 and 8 GPUs, and both gradients at full size
  contraction  [M,K,1] x [1,K,N] (Tensor.convDot) on the tensor-core and the FMA families
"""
from __future__ import annotations

import ctypes as C
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import baseline_configs as B  # noqa: E402
from neureka_b200 import _lib as L  # noqa: E402
from neureka_b200.ndconf import NDConfiguration as ND  # noqa: E402


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


def _row(ms, nbytes, hbm, dev, **more):
    r = {"ms": ms, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm, "kernel": dev.last_kernel()}
    r.update(more)
    return r


class Env:
    def __init__(self, dev, hbm_peak_gbs, small):
        self.dev, self.ctx, self.hbm, self.small = dev, dev.ctx, hbm_peak_gbs, small
        self._peaks = None

    @property
    def fma_peaks(self):
        """measured FMA ceilings (register-resident loop): denominators for the FMA-bound kernels"""
        if self._peaks is None:
            self._peaks = {}
            for name, dt in (("fp32", L.NK_F32), ("fp64", L.NK_F64)):
                v = C.c_double(0)
                L.check(L.lib.nk_measure_fma_peak(self.ctx, dt, C.byref(v)), self.ctx)
                self._peaks[name] = v.value
        return self._peaks


def sec_fma_peaks(e: Env):
    return {"measured_fma_peak_tflops": dict(e.fma_peaks)}


def sec_cfg1(e: Env):
    dev, ctx = e.dev, e.ctx
    a_h, k_h = B.cfg1_inputs()
    a, k, o = _Buf(dev, np.float32, 256 * 256, a_h), _Buf(dev, np.float32, 25, k_h), _Buf(dev, np.float32, 252 * 252)
    ca, pa = _cfg([256, 256]); ck, pk = _cfg([5, 5]); co, po = _cfg([252, 252])
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 2, o.buf, po, a.buf, pa, k.buf, pk, -1), ctx), 5, 200)
    out = {"us_per_launch": ms * 1e3, "gflops": 3175200 / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel(),
           "note": "0.5 MB problem, L2 resident: launch-latency bound"}
    for b in (a, k, o): b.free()
    return {"cfg1_conv2d_256x256_k5": out}


def sec_cfg2(e: Env):
    dev, ctx = e.dev, e.ctx
    n_in = 64 * 512 * 512
    a_h, k_h = B.cfg2_inputs()
    copies = [_Buf(dev, np.float32, n_in, a_h) for _ in range(4)]
    k = _Buf(dev, np.float32, 64 * 9, k_h)
    o = _Buf(dev, np.float32, 510 * 510)
    ca, pa = _cfg([64, 512, 512]); ck, pk = _cfg([64, 3, 3]); co, po = _cfg([1, 510, 510])
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 3, o.buf, po, copies[i % 4].buf, pa, k.buf, pk, -1), ctx), 4, 20)
    out = _row(ms, 68151568, e.hbm, dev, gflops=299635200 / (ms * 1e-3) / 1e9,
               note="4 rotating input copies (256 MiB) so that L2 cannot serve the reads")
    for b in copies + [k, o]: b.free()
    return {"cfg2_conv3d_64x512x512_k64x3x3": out}


def _cfg3_ops(e: Env, n, m, kk, reps):
    """The reference's op-by-op sequence for tanh(a*b+b) and the two reduced gradients, three full-size buffers."""
    dev, ctx = e.dev, e.ctx
    N = n * m * kk
    a_h, b_h = B.cfg3_inputs(n, m, kk)
    a, b = _Buf(dev, np.float32, n * kk, a_h), _Buf(dev, np.float32, m * kk, b_h)
    t2, y, g = (_Buf(dev, np.float32, N) for _ in range(3))
    ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
    ga, gb = _Buf(dev, np.float32, n * kk), _Buf(dev, np.float32, m * kk)
    small = 4.0 * (n * kk + m * kk)
    steps = [
        ("mul_broadcast", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t2.buf, po, a.buf, pa, b.buf, pb, -1), 4.0 * N + small),
        ("add_broadcast", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, y.buf, po, t2.buf, po, b.buf, pb, -1), 8.0 * N + 4.0 * m * kk),
        ("tanh", lambda i: L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g.buf, po, y.buf, po, -1), 8.0 * N),
        ("tanh_derivative", lambda i: L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g.buf, po, y.buf, po, 0), 8.0 * N),
        ("relu", lambda i: L.lib.nk_unary(ctx, L.FUN["relu"], L.NK_F32, 3, t2.buf, po, y.buf, po, -1), 8.0 * N),
        ("grad_a_reduce", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga.buf, pa, b.buf, pb, g.buf, po, 0), 4.0 * N + small),
        ("grad_b_reduce", lambda i: L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, gb.buf, pb, a.buf, pa, g.buf, po, 0), 4.0 * N + small),
    ]
    r = {}
    total = 0.0
    for name, fn, nbytes in steps:
        ms = _time(dev, lambda i, fn=fn: L.check(fn(i), ctx), 3, reps)
        if name != "relu":
            total += ms
        r[name] = _row(ms, nbytes, e.hbm, dev)
    r["forward_plus_backward_ms"] = total
    for bb in (a, b, t2, y, g, ga, gb): bb.free()
    return r


def sec_cfg3(e: Env):
    if e.small:   # 2^29 outputs, 2 GiB per tensor
        return {"cfg3_broadcast_tanh_1024x512x1024": _cfg3_ops(e, 1024, 512, 1024, 3)}
    r = _cfg3_ops(e, 2048, 1024, 1024, 4)
    r["tanh"]["note"] = "F32 tanh is defined by the reference as a double-precision formula evaluated per element, then cast"
    return {"cfg3_broadcast_tanh_2048x1024x1024": r}


def sec_cfg3_full(e: Env):
    """2^33 outputs: 4096*2048*1024 elements overflow Java's int sizes, so the reference itself cannot hold this tensor;
    here every intermediate is one 32 GiB buffer (64-bit offsets throughout). Needs ~100 GiB free."""
    if e.small or e.dev.props.total_mem_bytes < 150 * (1 << 30):
        return {}
    try:
        r = _cfg3_ops(e, 4096, 2048, 1024, 2)
        r["note"] = "2^33 F32 outputs per intermediate (32 GiB each); beyond the reference's int-sized tensors"
        return {"cfg3_full_size_4096x2048x1024": r}
    except Exception as ex:   # a side measurement must not take the others down
        return {"cfg3_full_size_4096x2048x1024": {"error": repr(ex)}}


def sec_cfg3_fused(e: Env):
    """cfg3 forward as ONE run-time compiled kernel (no 32 GiB intermediates)."""
    dev, ctx = e.dev, e.ctx
    try:
        r = {}
        h, h2 = C.c_void_p(), C.c_void_p()
        L.check(L.lib.nk_fused_compile(ctx, L.NK_F32, 2, b"f_tanh(op_add(op_mul(x0,x1),x1))", C.byref(h)), ctx)
        L.check(L.lib.nk_fused_compile(ctx, L.NK_F32, 2, b"op_add(op_mul(x0,x1),x1)", C.byref(h2)), ctx)
        sizes = (("1024x512x1024", (1024, 512, 1024)),) if e.small else (("2048x1024x1024", (2048, 1024, 1024)), ("4096x2048x1024_full_size", (4096, 2048, 1024)))
        for name, (n, m, kk) in sizes:
            N = n * m * kk
            if dev.props.total_mem_bytes < N * 4 + (8 << 30):
                continue
            a_h, b_h = B.cfg3_inputs(n, m, kk)
            a, b, y = _Buf(dev, np.float32, n * kk, a_h), _Buf(dev, np.float32, m * kk, b_h), _Buf(dev, np.float32, N)
            ca, pa = _cfg([n, 1, kk]); cb, pb = _cfg([1, m, kk]); co, po = _cfg([n, m, kk])
            bufs = (C.c_void_p * 2)(a.buf, b.buf)
            cfgs = (C.POINTER(C.c_int32) * 2)(pa, pb)
            nbytes = 4.0 * (N + n * kk + m * kk)
            ms2 = _time(dev, lambda i: L.check(L.lib.nk_fused_run(ctx, h2, 3, y.buf, po, bufs, cfgs), ctx), 3, 5)
            ms = _time(dev, lambda i: L.check(L.lib.nk_fused_run(ctx, h, 3, y.buf, po, bufs, cfgs), ctx), 3, 5)
            r[name] = {"tanh_affine_ms": ms, "tanh_affine_gbs": nbytes / (ms * 1e-3) / 1e9, "tanh_affine_frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / e.hbm,
                       "affine_only_ms": ms2, "affine_only_gbs": nbytes / (ms2 * 1e-3) / 1e9, "affine_only_frac_of_hbm_peak": nbytes / (ms2 * 1e-3) / 1e9 / e.hbm,
                       "kernel": dev.last_kernel()}
            for bb in (a, b, y): bb.free()
        r["note"] = "tanh(i0*i1+i1) / i0*i1+i1 in one pass: 24 MiB read, the result written once"
        L.lib.nk_fused_free(h); L.lib.nk_fused_free(h2)
        return {"cfg3_fused_forward": r}
    except Exception as ex:
        return {"cfg3_fused_forward": {"error": repr(ex)}}


def sec_contraction(e: Env):
    """Contraction-shaped `x` (Tensor.convDot: [M,K,1] x [1,K,N])."""
    dev, ctx = e.dev, e.ctx
    try:
        r = {}
        cases = (("f32_4096", L.NK_F32, np.float32, 4096, "fp32"),) if e.small else (
            ("f32_4096", L.NK_F32, np.float32, 4096, "fp32"), ("f32_8192", L.NK_F32, np.float32, 8192, "fp32"),
            ("f64_2048", L.NK_F64, np.float64, 2048, "fp64"), ("f32_1024", L.NK_F32, np.float32, 1024, "fp32"))
        for name, dt, npdt, n, fma_peak in cases:
            rng = np.random.default_rng(5)
            A = _Buf(dev, npdt, n * n, rng.standard_normal(n * n).astype(npdt))
            Bm = _Buf(dev, npdt, n * n, rng.standard_normal(n * n).astype(npdt))
            O = _Buf(dev, npdt, n * n)
            c1, p1 = _cfg([n, n, 1]); c2, p2 = _cfg([1, n, n]); c0, p0 = _cfg([n, 1, n])
            flops = 2.0 * n * n * n
            ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, dt, 3, O.buf, p0, A.buf, p1, Bm.buf, p2, -1), ctx), 3, 5)
            r[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "kernel": dev.last_kernel(),
                       "frac_of_measured_fma_peak": flops / (ms * 1e-3) / 1e12 / e.fma_peaks[fma_peak]}
            if not e.small and dt == L.NK_F32:   # the FMA family on the same call, for scale
                dev.set_conv_path(L.NK_CONV_GEMM)
                ms_f = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, dt, 3, O.buf, p0, A.buf, p1, Bm.buf, p2, -1), ctx), 3, 3)
                r[name]["fma_family_ms"] = ms_f
                r[name]["fma_family_kernel"] = dev.last_kernel()
                dev.set_conv_path(L.NK_CONV_AUTO)
            for bb in (A, Bm, O): bb.free()
        return {"contraction_MxKx1_x_1xKxN": r}
    except Exception as ex:
        dev.set_conv_path(L.NK_CONV_AUTO)
        return {"contraction_MxKx1_x_1xKxN": {"error": repr(ex)}}


def sec_cfg5_slabs(e: Env):
    """cfg5's forward pass on the slabs a rank holds at 4 and 8 GPUs (what bounds the multi-GPU rows)."""
    dev, ctx = e.dev, e.ctx
    try:
        r = {}
        for name, rows in (("one_of_8_ranks_260_rows", 260), ("one_of_4_ranks_515_rows", 515), ("one_of_2_ranks_1026_rows", 1026)):
            Bn, Cn, W, KH = 8, 32, 2048, 5
            img = _Buf(dev, np.float32, Bn * Cn * rows * W)
            L.check(L.lib.nk_fill(ctx, img.buf, C.c_double(0.5), 0, Bn * Cn * rows * W), ctx)
            ker = _Buf(dev, np.float32, Cn * KH * KH, B.cfg5_kernel())
            o = _Buf(dev, np.float32, Bn * (rows - 4) * (W - 4))
            ci, pi_ = _cfg([Bn, Cn, rows, W]); ckk, pkk = _cfg([1, Cn, KH, KH]); co_, po_ = _cfg([Bn, 1, rows - 4, W - 4])
            ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, o.buf, po_, img.buf, pi_, ker.buf, pkk, -1), ctx), 3, 20)
            flops = 2.0 * Bn * (rows - 4) * (W - 4) * Cn * KH * KH
            r[name] = {"ms": ms, "tflops": flops / (ms * 1e-3) / 1e12, "kernel": dev.last_kernel()}
            for bb in (img, ker, o): bb.free()
            if e.small:
                break
        return {"cfg5_forward_on_one_rank_slab": r}
    except Exception as ex:
        return {"cfg5_forward_on_one_rank_slab": {"error": repr(ex)}}


def sec_cfg5_gradients(e: Env):
    """Gradients of cfg5's convolution (error uniform [-1,1], seed 9); --small: a quarter-height image (1 GiB)."""
    dev, ctx = e.dev, e.ctx
    try:
        Bn, Cn, H, W, KH = 8, 32, (512 if e.small else 2048), 2048, 5
        OH, OW = H - KH + 1, W - KH + 1
        from neureka_b200 import jrand
        img = _Buf(dev, np.float32, Bn * Cn * H * W)
        L.check(L.lib.nk_fill(ctx, img.buf, C.c_double(0.5), 0, Bn * Cn * H * W), ctx)
        err = _Buf(dev, np.float32, Bn * OH * OW, jrand.fill(np.zeros(Bn * OH * OW, dtype=np.float32), jrand.UNIFORM, 9, -1.0, 1.0))
        ker = _Buf(dev, np.float32, Cn * KH * KH, B.cfg5_kernel())
        gimg, gker = _Buf(dev, np.float32, Bn * Cn * H * W), _Buf(dev, np.float32, Cn * KH * KH)
        ci, pi_ = _cfg([Bn, Cn, H, W]); ce, pe = _cfg([Bn, 1, OH, OW]); ckk, pkk = _cfg([1, Cn, KH, KH])
        flops = 2.0 * Bn * OH * OW * Cn * KH * KH
        nbytes = 4.0 * (Bn * Cn * H * W + Bn * OH * OW + Cn * KH * KH)
        r = {}
        ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gimg.buf, pi_, ker.buf, pkk, err.buf, pe, 0), ctx), 3, 10)
        r["grad_image"] = _row(ms, nbytes, e.hbm, dev, tflops=flops / (ms * 1e-3) / 1e12, frac_of_measured_fma_peak=flops / (ms * 1e-3) / 1e12 / e.fma_peaks["fp32"])
        ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, gker.buf, pkk, img.buf, pi_, err.buf, pe, 0), ctx), 3, 10)
        r["grad_kernel"] = _row(ms, nbytes, e.hbm, dev, tflops=flops / (ms * 1e-3) / 1e12, frac_of_measured_fma_peak=flops / (ms * 1e-3) / 1e12 / e.fma_peaks["fp32"])
        for bb in (img, err, ker, gimg, gker): bb.free()
        return {"cfg5_gradients_quarter_height" if e.small else "cfg5_gradients": r}
    except Exception as ex:
        return {"cfg5_gradients": {"error": repr(ex)}}


def sec_cfg4(e: Env):
    dev, ctx = e.dev, e.ctx
    v_h, k_h = B.cfg4_inputs()
    v, k = _Buf(dev, np.float64, 128 ** 3, v_h), _Buf(dev, np.float64, 343, k_h)
    yb = _Buf(dev, np.float64, 122 ** 3)
    gv, gk = _Buf(dev, np.float64, 128 ** 3), _Buf(dev, np.float64, 343)
    cv, pv = _cfg([128] * 3); ck, pk = _cfg([7] * 3); cy, py = _cfg([122] * 3)
    flops = 1245671728.0
    r = {}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, yb.buf, py, v.buf, pv, k.buf, pk, -1), ctx), 3, 10)
    r["forward"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    # gradients for error = y itself (any error tensor does): XConvRight(error, other, zeros) -> (drain, other, error), d = 0
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, gv.buf, pv, k.buf, pk, yb.buf, py, 0), ctx), 3, 10)
    r["grad_volume"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    ms = _time(dev, lambda i: L.check(L.lib.nk_conv(ctx, L.NK_F64, 3, gk.buf, pk, v.buf, pv, yb.buf, py, 0), ctx), 3, 10)
    r["grad_kernel"] = {"ms": ms, "gflops": flops / (ms * 1e-3) / 1e9, "kernel": dev.last_kernel()}
    for v_ in r.values():
        v_["frac_of_fp64_fma_peak"] = v_["gflops"] / 1e3 / e.fma_peaks["fp64"]
    for bb in (v, k, yb, gv, gk): bb.free()
    return {"cfg4_conv3d_f64_128_k7": r}


def sec_cfg5_group(e: Env):
    """cfg5's forward pass through the in-process device group (nk_conv_sharded) on every visible GPU: one host thread,
    one context per GPU, slabs resident, result assembled in the first GPU's memory. Needs two GPUs or more."""
    from neureka_b200.device import CudaDevice
    from neureka_b200.sharding import plan_slabs
    n = CudaDevice.count()
    if n < 2:
        return {"cfg5_in_process_group": {"skipped": "one GPU visible"}}
    Bn, Cn, H, W, KH = 8, 32, 2048, 2048, 5
    grp = C.c_void_p()
    L.check(L.lib.nk_group_open((C.c_int32 * n)(*range(n)), n, C.byref(grp)))
    try:
        ctxs = []
        for i in range(n):
            c = C.c_void_p()
            L.check(L.lib.nk_group_ctx(grp, i, C.byref(c)))
            ctxs.append(c)
        slabs = plan_slabs(H - KH + 1, n, KH - 1)
        k_h = np.ascontiguousarray(B.cfg5_kernel(), dtype=np.float32)
        sb, kb = [], []
        for i, s in enumerate(slabs):
            rows = s.in_hi - s.in_lo
            b_, k_ = C.c_void_p(), C.c_void_p()
            L.check(L.lib.nk_alloc(ctxs[i], L.NK_F32, Bn * Cn * rows * W, C.byref(b_)), ctxs[i])
            L.check(L.lib.nk_fill(ctxs[i], b_, C.c_double(0.5), 0, Bn * Cn * rows * W), ctxs[i])
            L.check(L.lib.nk_alloc(ctxs[i], L.NK_F32, k_h.size, C.byref(k_)), ctxs[i])
            L.check(L.lib.nk_write(ctxs[i], k_, k_h.ctypes.data_as(C.c_void_p), 0, 0, k_h.size), ctxs[i])
            sb.append(b_); kb.append(k_)
        n_out = Bn * (H - KH + 1) * (W - KH + 1)
        out = C.c_void_p()
        L.check(L.lib.nk_alloc(ctxs[0], L.NK_F32, n_out, C.byref(out)), ctxs[0])
        ish, ksh = (C.c_int64 * 4)(Bn, Cn, H, W), (C.c_int64 * 4)(1, Cn, KH, KH)
        sl, kl = (C.c_void_p * n)(*sb), (C.c_void_p * n)(*kb)
        run = lambda: L.check(L.lib.nk_conv_sharded(grp, L.NK_F32, 4, ish, ksh, 2, sl, kl, out), ctxs[0])
        for _ in range(3):
            run()
        for c in ctxs:
            L.check(L.lib.nk_sync(c), c)
        reps = 20
        L.check(L.lib.nk_timer_begin(ctxs[0]), ctxs[0])   # the first member's stream waits for every push: its timer sees whole passes
        for _ in range(reps):
            run()
        ms = C.c_float(0)
        L.check(L.lib.nk_timer_end(ctxs[0], C.byref(ms)), ctxs[0])
        for c in ctxs:
            L.check(L.lib.nk_sync(c), c)
        ms = float(ms.value) / reps
        flops = 2.0 * n_out * Cn * KH * KH
        for i in range(n):
            L.lib.nk_free(ctxs[i], sb[i]); L.lib.nk_free(ctxs[i], kb[i])
        L.lib.nk_free(ctxs[0], out)
        return {"cfg5_in_process_group": {"n_gpus": n, "ms_per_pass": ms, "tflops_total": flops / (ms * 1e-3) / 1e12,
                                          "note": "one host thread, nk_conv_sharded; pushes of pass k overlap pass k+1"}}
    finally:
        L.check(L.lib.nk_group_close(grp))


SECTIONS = {
    "fma_peaks": sec_fma_peaks, "cfg1": sec_cfg1, "cfg2": sec_cfg2, "cfg3": sec_cfg3, "cfg3_fused": sec_cfg3_fused,
    "cfg3_full": sec_cfg3_full, "contraction": sec_contraction, "cfg5_slabs": sec_cfg5_slabs,
    "cfg5_gradients": sec_cfg5_gradients, "cfg4": sec_cfg4, "cfg5_group": sec_cfg5_group,
}


def run_extra(dev, hbm_peak_gbs: float, only=None, small: bool = False) -> dict:
    e = Env(dev, hbm_peak_gbs, small)
    out = {}
    for name, fn in SECTIONS.items():
        if only and name not in only:
            continue
        if not only and name == "cfg5_group":   # uses every visible GPU: only when asked for by name
            continue
        out.update(fn(e))
    return out


if __name__ == "__main__":
    import argparse
    from neureka_b200.device import CudaDevice
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--small", action="store_true")
    a = ap.parse_args()
    peak = 6558.7
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            peak = float(json.load(f)["hbm_gbs"])
    only = [s for s in a.only.split(",") if s]
    for s in only:
        if s not in SECTIONS:
            raise SystemExit(f"unknown section {s}; known: {', '.join(SECTIONS)}")
    print(json.dumps(run_extra(CudaDevice.get(0), peak, only, a.small), indent=1))
