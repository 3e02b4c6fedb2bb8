"""Shared helpers of the parity tests: host arrays + NDConfigurations -> oracle result / CUDA result."""
import ctypes as C

import numpy as np

from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND


class DevArray:
    """A raw device buffer driven straight through the C ABI (no Tensor layer in between)."""

    def __init__(self, device, host: np.ndarray):
        self.device = device
        self.dtype = host.dtype
        self.n = host.size
        self.buf = C.c_void_p()
        dt = L.NK_F32 if host.dtype == np.float32 else L.NK_F64
        self.nk_dtype = dt
        L.check(L.lib.nk_alloc(device.ctx, dt, host.size, C.byref(self.buf)), device.ctx)
        h = np.ascontiguousarray(host)
        L.check(L.lib.nk_write(device.ctx, self.buf, h.ctypes.data_as(C.c_void_p), 0, 0, h.size), device.ctx)

    def read(self) -> np.ndarray:
        out = np.empty(self.n, dtype=self.dtype)
        L.check(L.lib.nk_read(self.device.ctx, self.buf, out.ctypes.data_as(C.c_void_p), 0, self.n), self.device.ctx)
        return out

    def free(self):
        if self.buf:
            L.lib.nk_free(self.device.ctx, self.buf)
            self.buf = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def cfgp(conf):
    arr = conf.as_inline_array() if isinstance(conf, ND) else np.ascontiguousarray(conf, dtype=np.int32)
    return arr, arr.ctypes.data_as(C.POINTER(C.c_int32))


def gpu_conv(device, drn, c0, a, c1, b, c2, d=-1, path=L.NK_CONV_AUTO):
    """nk_conv on copies of the host arrays; returns the drain's data array."""
    D, A, B = DevArray(device, drn), DevArray(device, a), DevArray(device, b)
    k0, p0 = cfgp(c0); k1, p1 = cfgp(c1); k2, p2 = cfgp(c2)
    device.set_conv_path(path)
    try:
        L.check(L.lib.nk_conv(device.ctx, D.nk_dtype, len(k0) // 5, D.buf, p0, A.buf, p1, B.buf, p2, d), device.ctx)
        out = D.read()
    finally:
        device.set_conv_path(L.NK_CONV_AUTO)
        D.free(); A.free(); B.free()
    return out


CONV_TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


def assert_conv_close(got, ref, scale, what=""):
    """The convolution tolerance, per element and with no extra factor: |got - ref| <= tol * sum|a||b| (tol = 1e-5 for
    F32, 1e-12 for F64; `scale` is the same sum taken over absolute values, the magnitude any summation order is
    measured against). Returns the largest error / bound ratio seen."""
    dt = np.dtype(got.dtype)
    err = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    bound = CONV_TOL[dt] * np.maximum(np.abs(scale).astype(np.float64), np.finfo(dt).tiny)
    worst = int(np.argmax(err / bound))
    assert np.all(err <= bound), f"{what}: err {err.flat[worst]:.3e} > bound {bound.flat[worst]:.3e} at {worst}"
    return float((err / bound).max())


def gpu_call3(fn, device, op, drn, c0, a, c1, b, c2, d=-1):
    D, A, B = DevArray(device, drn), DevArray(device, a), DevArray(device, b)
    k0, p0 = cfgp(c0); k1, p1 = cfgp(c1); k2, p2 = cfgp(c2)
    try:
        L.check(fn(device.ctx, op, D.nk_dtype, len(k0) // 5, D.buf, p0, A.buf, p1, B.buf, p2, d), device.ctx)
        return D.read()
    finally:
        D.free(); A.free(); B.free()


def gpu_unary(device, fun, drn, c0, a, c1, d=-1):
    D, A = DevArray(device, drn), DevArray(device, a)
    k0, p0 = cfgp(c0); k1, p1 = cfgp(c1)
    try:
        L.check(L.lib.nk_unary(device.ctx, fun, D.nk_dtype, len(k0) // 5, D.buf, p0, A.buf, p1, d), device.ctx)
        return D.read()
    finally:
        D.free(); A.free()


def gpu_scalar(device, op, drn, c0, a, c1, value, d=-1):
    D, A = DevArray(device, drn), DevArray(device, a)
    k0, p0 = cfgp(c0); k1, p1 = cfgp(c1)
    try:
        L.check(L.lib.nk_scalar_binary(device.ctx, op, D.nk_dtype, len(k0) // 5, D.buf, p0, A.buf, p1, float(value), d), device.ctx)
        return D.read()
    finally:
        D.free(); A.free()


def ulp_diff(x: np.ndarray, y: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between two float arrays of the same dtype, in exact integer
    arithmetic (NaN == NaN counts as 0; distances beyond 2**62 saturate)."""
    assert x.dtype == y.dtype
    it = np.int32 if x.dtype == np.float32 else np.int64
    xi = x.view(it).astype(np.int64)
    yi = y.view(it).astype(np.int64)
    lo = np.int64(np.iinfo(it).min)
    # map the sign-magnitude float ordering onto a monotone integer line: negative floats -> -(magnitude)
    xm = np.where(xi < 0, lo - xi, xi)
    ym = np.where(yi < 0, lo - yi, yi)
    same_side = (xm >= 0) == (ym >= 0)
    near = np.abs(np.where(same_side, xm - ym, 0))
    far = np.minimum(np.abs(xm.astype(np.float64)) + np.abs(ym.astype(np.float64)), 2.0 ** 62).astype(np.int64)
    dist = np.where(same_side, near, far)
    both_nan = np.isnan(x) & np.isnan(y)
    return np.where(both_nan, 0, dist)


def rand_view(rng, shape, kind):
    """A view of `shape` of kind 'dense' | 'sliced' | 'strided' | 'colmajor' | 'permuted' and the size of the
    data array it needs."""
    shape = tuple(int(s) for s in shape)
    rank = len(shape)
    if kind == "dense":
        c = ND.of_shape(shape)
        return c, c.required_elements()
    if kind == "colmajor":
        from neureka_b200.ndconf import Layout
        c = ND.of_shape(shape, Layout.COLUMN_MAJOR)
        return c, c.required_elements()
    if kind == "permuted":
        perm = list(rng.permutation(rank))
        parent_shape = [0] * rank
        for new_axis, old_axis in enumerate(perm):
            parent_shape[old_axis] = shape[new_axis]
        c = ND.of_shape(parent_shape).reshaped(perm)
        assert c.shape == shape
        return c, c.required_elements()
    offs = [int(rng.integers(0, 3)) for _ in range(rank)]
    if kind == "sliced":
        spread = [1] * rank
    else:
        spread = [int(rng.integers(1, 4)) if s > 1 else 1 for s in shape]
    parent = [offs[k] + (shape[k] - 1) * spread[k] + 1 + int(rng.integers(0, 2)) for k in range(rank)]
    c = ND.of_shape(parent).sliced(shape, offs, spread)
    return c, ND.of_shape(parent).required_elements()
