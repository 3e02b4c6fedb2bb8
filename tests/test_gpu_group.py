"""The in-process device group (nk_group_*, nk_conv_sharded): one host process drives several contexts, the halo-split
forward convolution runs a slab per member and the result is assembled in the first member's memory. Compared bit for
bit with the same convolution on one context. With one GPU the group is two contexts on the same ordinal (two streams);
with two or more GPUs a second case uses distinct devices and their peer copies."""
import ctypes as C

import numpy as np
import pytest

from neureka_b200 import _lib as L
from neureka_b200.device import CudaDevice
from neureka_b200.ndconf import NDConfiguration as ND
from neureka_b200.sharding import plan_slabs

pytestmark = pytest.mark.gpu


def _cfg(shape):
    a = ND.of_shape(shape).as_inline_array()
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def _run_group(ordinals, dt, a_shape, k_shape, dim, repeats=3):
    npdt = np.float32 if dt == L.NK_F32 else np.float64
    rng = np.random.default_rng(7)
    a = rng.standard_normal(a_shape).astype(npdt)
    k = rng.standard_normal(k_shape).astype(npdt)
    o_shape = [abs(x - y) + 1 for x, y in zip(a_shape, k_shape)]
    n = len(ordinals)
    grp = C.c_void_p()
    L.check(L.lib.nk_group_open((C.c_int32 * n)(*ordinals), n, C.byref(grp)))
    try:
        size = C.c_int32()
        L.check(L.lib.nk_group_size(grp, C.byref(size)))
        assert size.value == n
        ctxs = []
        for i in range(n):
            c = C.c_void_p()
            L.check(L.lib.nk_group_ctx(grp, i, C.byref(c)))
            ctxs.append(c)
        slabs = plan_slabs(o_shape[dim], n, k_shape[dim] - 1)
        slab_bufs, kern_bufs = [], []
        for i, s in enumerate(slabs):
            idx = [slice(None)] * len(a_shape)
            idx[dim] = slice(s.in_lo, max(s.in_hi, s.in_lo + 1))
            part = np.ascontiguousarray(a[tuple(idx)])
            sb, kb = C.c_void_p(), C.c_void_p()
            L.check(L.lib.nk_alloc(ctxs[i], dt, part.size, C.byref(sb)), ctxs[i])
            L.check(L.lib.nk_write(ctxs[i], sb, part.ctypes.data_as(C.c_void_p), 0, 0, part.size), ctxs[i])
            L.check(L.lib.nk_alloc(ctxs[i], dt, k.size, C.byref(kb)), ctxs[i])
            L.check(L.lib.nk_write(ctxs[i], kb, k.ctypes.data_as(C.c_void_p), 0, 0, k.size), ctxs[i])
            slab_bufs.append(sb); kern_bufs.append(kb)
        n_out = int(np.prod(o_shape))
        out = C.c_void_p()
        L.check(L.lib.nk_alloc(ctxs[0], dt, n_out, C.byref(out)), ctxs[0])
        L.check(L.lib.nk_fill(ctxs[0], out, C.c_double(777.0), 0, n_out), ctxs[0])
        ish, ksh = (C.c_int64 * len(a_shape))(*a_shape), (C.c_int64 * len(k_shape))(*k_shape)
        sl, kl = (C.c_void_p * n)(*slab_bufs), (C.c_void_p * n)(*kern_bufs)
        got = np.empty(n_out, dtype=npdt)
        for _ in range(repeats):   # repeated calls rotate the local slabs; each must leave the complete result
            st = L.lib.nk_conv_sharded(grp, dt, len(a_shape), ish, ksh, dim, sl, kl, out)
            L.check(st, ctxs[0])
            L.check(L.lib.nk_read(ctxs[0], out, got.ctypes.data_as(C.c_void_p), 0, n_out), ctxs[0])   # the owner's stream sees it assembled
        # the same convolution on one context
        dev = CudaDevice.get(ordinals[0])
        A, K, O = C.c_void_p(), C.c_void_p(), C.c_void_p()
        for buf, arr in ((A, a), (K, k)):
            L.check(L.lib.nk_alloc(dev.ctx, dt, arr.size, C.byref(buf)), dev.ctx)
            L.check(L.lib.nk_write(dev.ctx, buf, np.ascontiguousarray(arr).ctypes.data_as(C.c_void_p), 0, 0, arr.size), dev.ctx)
        L.check(L.lib.nk_alloc(dev.ctx, dt, n_out, C.byref(O)), dev.ctx)
        (_, pa), (_, pk), (_, po) = _cfg(a_shape), _cfg(k_shape), _cfg(o_shape)
        ka, kk, ko = _cfg(a_shape), _cfg(k_shape), _cfg(o_shape)
        L.check(L.lib.nk_conv(dev.ctx, dt, len(a_shape), O, ko[1], A, ka[1], K, kk[1], -1), dev.ctx)
        want = np.empty(n_out, dtype=npdt)
        L.check(L.lib.nk_read(dev.ctx, O, want.ctypes.data_as(C.c_void_p), 0, n_out), dev.ctx)
        for buf in (A, K, O):
            L.lib.nk_free(dev.ctx, buf)
        for i in range(n):
            L.lib.nk_free(ctxs[i], slab_bufs[i]); L.lib.nk_free(ctxs[i], kern_bufs[i])
        L.lib.nk_free(ctxs[0], out)
        return got, want
    finally:
        L.check(L.lib.nk_group_close(grp))


@pytest.mark.parametrize("dt", [L.NK_F32, L.NK_F64])
@pytest.mark.parametrize("parts", [1, 2, 3])
def test_sharded_convolution_on_one_gpu_equals_the_unsharded_one(device, dt, parts):
    got, want = _run_group([0] * parts, dt, [3, 6, 150, 260], [1, 6, 5, 5], 2)
    assert np.array_equal(got, want)


def test_a_split_along_a_batch_like_dim_needs_no_halo(device):
    got, want = _run_group([0, 0], L.NK_F32, [6, 4, 40, 132], [1, 4, 3, 3], 0)
    assert np.array_equal(got, want)


def test_sharded_convolution_across_two_gpus(device):
    if CudaDevice.count() < 2:
        pytest.skip("needs two GPUs")
    got, want = _run_group([0, 1], L.NK_F32, [4, 6, 300, 520], [1, 6, 5, 5], 2)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("ordinals", [[0, 0], [0, 1]])
def test_sharded_convolution_when_the_channel_split_differs(device, ordinals):
    """With 8 or more channels and fewer tiles than resident CTAs the tiled family splits the channel range over several
    CTAs and adds their partial tiles in part order. Whether it does depends on the tile count, so a slab (half the
    rows) and the whole image may be summed in a different order: equal to rounding, not necessarily bit for bit."""
    if max(ordinals) >= CudaDevice.count():
        pytest.skip("needs two GPUs")
    got, want = _run_group(ordinals, L.NK_F32, [4, 8, 300, 520], [1, 8, 5, 5], 2)
    assert np.abs(got - want).max() <= 1e-5 * 8 * 25 * 3.0 * 3.0    # 1e-5 x (terms x a bound on |a||b| of unit normals)
    assert np.abs(got - want).max() <= 2e-4


def test_group_argument_errors(device):
    grp = C.c_void_p()
    assert L.lib.nk_group_open((C.c_int32 * 1)(99), 1, C.byref(grp)) == L.NK_ERR_BAD_ARG
    L.check(L.lib.nk_group_open((C.c_int32 * 2)(0, 0), 2, C.byref(grp)))
    try:
        c0 = C.c_void_p()
        L.check(L.lib.nk_group_ctx(grp, 0, C.byref(c0)))
        assert L.lib.nk_group_ctx(grp, 5, C.byref(c0)) == L.NK_ERR_BAD_ARG
        out = C.c_void_p()
        L.check(L.lib.nk_alloc(c0, L.NK_F32, 16, C.byref(out)), c0)
        ish, ksh = (C.c_int64 * 2)(8, 8), (C.c_int64 * 2)(8, 3)
        bufs = (C.c_void_p * 2)(out, out)
        # dim 0 has equal extents (summed away): it cannot be halo-split
        assert L.lib.nk_conv_sharded(grp, L.NK_F32, 2, ish, ksh, 0, bufs, bufs, out) == L.NK_ERR_BAD_ARG
        # the result does not fit the buffer
        ish2 = (C.c_int64 * 2)(64, 64)
        assert L.lib.nk_conv_sharded(grp, L.NK_F32, 2, ish2, ksh, 1, bufs, bufs, out) == L.NK_ERR_BOUNDS
        L.lib.nk_free(c0, out)
    finally:
        L.check(L.lib.nk_group_close(grp))
