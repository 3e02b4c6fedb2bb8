"""Parity of the broadcast / elementwise / scalar kernels with the CPU oracle. Tolerance: at most 1 ulp
(the task's bound for elementwise ops); arithmetic-only functions are required to be bit-exact."""
import ctypes as C

import numpy as np
import pytest

from helpers import DevArray, cfgp, gpu_call3, gpu_scalar, gpu_unary, rand_view, ulp_diff
from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND

pytestmark = pytest.mark.gpu
EXACT_FUNS = {"abs", "idy", "quad", "relu", "fast_gaus", "softsign", "gasu", "fast_tanh", "sqrt"}
OPS = ["+", "-", "*", "/", "%", "**"]


def _inputs(rng, n, dt, fun=None, positive=False):
    x = (rng.standard_normal(n) * 3).astype(dt)
    if positive or fun in ("ln", "log10", "sqrt", "cbrt"):
        x = np.abs(x) + dt(0.01)
    return x


def _assert_close(got, ref, max_ulp, what, x=None):
    """F32: at most `max_ulp` ulp, strictly (the F32 definitions evaluate in double and round once).
    F64 transcendental results (max_ulp > 0): the reference's own building blocks (java.lang.Math exp/log/pow/
    sin/cos/cbrt) are only specified to 1-2 ulp and formulas such as 2/(1+exp(-2x))-1 amplify that last bit by
    cancellation, so two conforming math libraries differ by more than 1 ulp of the *result*; the bound used is
    2 ulp of the result plus 4 ulp of the magnitude of the intermediates those formulas cancel: 1.0, or 3x^2 for
    the derivative of gatu (3x^2 * (1 - tanh(x^3)^2))."""
    assert got.dtype == ref.dtype
    assert np.array_equal(np.isinf(got), np.isinf(ref)), what
    assert np.array_equal(np.isnan(got), np.isnan(ref)), what
    fin = np.isfinite(ref)
    d = ulp_diff(got, ref)
    if got.dtype == np.float64 and max_ulp > 0:
        scale = 1.0 if x is None else np.maximum(1.0, 3.0 * x.astype(np.float64) ** 2)
        ok = (d <= 2) | (np.abs(got - ref) <= 4 * np.finfo(np.float64).eps * scale)
        bad = fin & ~ok
        assert not bad.any(), f"{what}: {d[bad].max()} ulp at ref {ref[bad][0]!r} vs got {got[bad][0]!r}"
        return
    assert d[fin].max(initial=0) <= max_ulp, f"{what}: {d[fin].max()} ulp at {ref[fin][d[fin].argmax()]!r} vs {got[fin][d[fin].argmax()]!r}"


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("fun", L.FUN_IDS)
@pytest.mark.parametrize("d", [-1, 0])
def test_activation_functions(device, oracle, dt, fun, d):
    rng = np.random.default_rng(L.FUN[fun] * 2 + (d + 1))
    n = 10_007   # odd: exercises the vector tail
    x = _inputs(rng, n, dt, fun)
    x[:8] = np.asarray([0, 1, -1, 0.5, -0.5, 4, -4, 1e-3], dtype=dt) if fun not in ("ln", "log10", "sqrt", "cbrt") else x[:8]
    ref = np.zeros(n, dtype=dt)
    c = ND.of_shape([n])
    oracle.unary(fun, ref, c.as_inline_array(), x, c.as_inline_array(), d=d, threads=4)
    got = gpu_unary(device, L.FUN[fun], np.zeros(n, dtype=dt), c, x, c, d=d)
    _assert_close(got, ref, 0 if fun in EXACT_FUNS else 1, f"{fun} d={d} {np.dtype(dt)}", x=x)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_activation_on_views(device, oracle, dt):
    rng = np.random.default_rng(3)
    for kind0, kind1, shape in [("sliced", "strided", [7, 33]), ("dense", "permuted", [5, 6, 7]), ("strided", "colmajor", [4, 300]),
                                ("dense", "sliced", [3, 4, 260]), ("permuted", "dense", [6, 5])]:
        c0, n0 = rand_view(rng, shape, kind0)
        c1, n1 = rand_view(rng, shape, kind1)
        x = _inputs(rng, n1, dt)
        ref = np.full(n0, 5.0, dtype=dt)
        oracle.unary("tanh", ref, c0.as_inline_array(), x, c1.as_inline_array(), threads=2)
        got = gpu_unary(device, L.FUN["tanh"], np.full(n0, 5.0, dtype=dt), c0, x, c1)
        _assert_close(got, ref, 1, f"tanh on {kind0}/{kind1}")


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("op", OPS)
@pytest.mark.parametrize("d", [-1, 0, 1])
def test_bielementwise(device, oracle, dt, op, d):
    rng = np.random.default_rng(17)
    n = 4099
    a = _inputs(rng, n, dt, positive=(op == "**"))
    b = _inputs(rng, n, dt)
    b[np.abs(b) < 0.05] = dt(0.5)
    c = ND.of_shape([n])
    ref = np.zeros(n, dtype=dt)
    oracle.bielementwise(op, ref, c.as_inline_array(), a, c.as_inline_array(), b, c.as_inline_array(), d=d, threads=3)
    got = gpu_call3(L.lib.nk_binary, device, L.OPS[op], np.zeros(n, dtype=dt), c, a, c, b, c, d=d)
    _assert_close(got, ref, 1 if op in ("**", "/", "%") else 0, f"bielementwise {op} d={d}")


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_bielementwise_on_views(device, oracle, dt):
    rng = np.random.default_rng(19)
    for kinds, shape in [(("sliced", "sliced", "dense"), [9, 11]), (("dense", "permuted", "strided"), [4, 5, 6]), (("dense", "dense", "sliced"), [3, 512])]:
        (c0, n0), (c1, n1), (c2, n2) = (rand_view(rng, shape, k) for k in kinds)
        a, b = _inputs(rng, n1, dt), _inputs(rng, n2, dt)
        ref = np.zeros(n0, dtype=dt)
        oracle.bielementwise("*", ref, c0.as_inline_array(), a, c1.as_inline_array(), b, c2.as_inline_array())
        got = gpu_call3(L.lib.nk_binary, device, L.NK_OP_MUL, np.zeros(n0, dtype=dt), c0, a, c1, b, c2)
        _assert_close(got, ref, 0, f"mul on views {kinds}")


def test_golden_sliced_addition(device, kat):
    v = kat["sliced_addition"]
    data = np.resize(np.arange(3, 20, dtype=np.float64), 121)
    parent = ND.of_shape([11, 11])
    x, y = parent.sliced([9, 11], [1, 0], [1, 1]), parent.sliced([9, 11], [0, 0], [1, 1])
    got = gpu_call3(L.lib.nk_binary, device, L.NK_OP_ADD, np.zeros(99), ND.of_shape([9, 11]), data, x, data, y)
    assert got[:50].tolist() == [float(t) for t in v["first_50"]]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("op", OPS)
def test_broadcast_forward(device, oracle, dt, op):
    rng = np.random.default_rng(23)
    cases = [([1, 3], [2, 1]), ([6, 1, 130], [1, 5, 130]), ([4, 1, 7], [4, 5, 1]), ([3, 256], [1, 256]), ([2, 3, 4], [2, 3, 4]),
             ([1, 1, 1], [3, 2, 5]), ([8, 1, 512], [1, 4, 512])]
    for s1, s2 in cases:
        so = [max(x, y) for x, y in zip(s1, s2)]
        a = _inputs(rng, int(np.prod(s1)), dt, positive=(op == "**"))
        b = _inputs(rng, int(np.prod(s2)), dt)
        b[np.abs(b) < 0.05] = dt(0.5)
        c0, c1, c2 = ND.of_shape(so), ND.of_shape(s1), ND.of_shape(s2)
        ref = np.zeros(c0.size, dtype=dt)
        oracle.broadcast(op, ref, c0.as_inline_array(), a, c1.as_inline_array(), b, c2.as_inline_array(), threads=2)
        got = gpu_call3(L.lib.nk_broadcast, device, L.OPS[op], np.zeros(c0.size, dtype=dt), c0, a, c1, b, c2)
        _assert_close(got, ref, 1 if op in ("**", "/", "%") else 0, f"broadcast {op} {s1}x{s2}")


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_broadcast_golden_and_views(device, oracle, kat, dt):
    v = kat["broadcast_forward_mul"][0]
    got = gpu_call3(L.lib.nk_broadcast, device, L.NK_OP_MUL, np.zeros(6, dtype=dt), ND.of_shape(v["out_shape"]), np.asarray(v["a"], dtype=dt),
                    ND.of_shape(v["a_shape"]), np.asarray(v["b"], dtype=dt), ND.of_shape(v["b_shape"]))
    assert got.tolist() == [float(x) for x in v["out"]]
    w = kat["broadcast_backward_mul_both"][0]
    got = gpu_call3(L.lib.nk_broadcast, device, L.NK_OP_MUL_BOTH, np.zeros(3, dtype=dt), ND.of_shape(w["origin_shape"]), np.asarray(w["handle"], dtype=dt),
                    ND.of_shape(w["handle_shape"]), np.asarray(w["drain"], dtype=dt), ND.of_shape(w["drain_shape"]), d=0)
    assert got.tolist() == [float(x) for x in w["out"]]
    rng = np.random.default_rng(29)
    (c0, n0), (c1, n1), (c2, n2) = rand_view(rng, [5, 6, 140], "sliced"), rand_view(rng, [5, 1, 140], "strided"), rand_view(rng, [1, 6, 140], "permuted")
    a, b = _inputs(rng, n1, dt), _inputs(rng, n2, dt)
    ref = np.zeros(n0, dtype=dt)
    oracle.broadcast("+", ref, c0.as_inline_array(), a, c1.as_inline_array(), b, c2.as_inline_array())
    got = gpu_call3(L.lib.nk_broadcast, device, L.NK_OP_ADD, np.zeros(n0, dtype=dt), c0, a, c1, b, c2)
    _assert_close(got, ref, 0, "broadcast + on views")


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("op", ["+", "-", "*", "/", "**"])
@pytest.mark.parametrize("d", [0, 1])
def test_broadcast_backward_reduction(device, oracle, dt, op, d):
    """(origin, handle, drain): sum over the dims where the origin is smaller, in the CPU's summation order,
    hence bit-exact for + - * and within 1 ulp per term for the pow/div derivative formulas."""
    rng = np.random.default_rng(31)
    cases = [([1, 3], [2, 1], [2, 3]), ([4, 1, 33], [1, 5, 33], [4, 5, 33]), ([1, 5, 33], [4, 1, 33], [4, 5, 33]),
             ([1, 1, 6], [7, 8, 1], [7, 8, 6]), ([3, 4], [3, 4], [3, 4]), ([1], [9], [9]),
             # shapes that take the vectorised reduction (inner dim kept, multiple of the vector width)
             ([8, 1, 64], [1, 6, 64], [8, 6, 64]), ([1, 5, 64], [4, 1, 64], [4, 5, 64]), ([3, 1, 64], [1, 5, 1], [3, 5, 64]),
             ([1, 1, 128], [6, 7, 128], [6, 7, 128]), ([2, 1, 1, 32], [1, 3, 4, 32], [2, 3, 4, 32])]
    for s0, s1, s2 in cases:
        h = _inputs(rng, int(np.prod(s1)), dt, positive=(op == "**"))
        dr = _inputs(rng, int(np.prod(s2)), dt)
        dr[np.abs(dr) < 0.05] = dt(0.5)
        c0, c1, c2 = ND.of_shape(s0), ND.of_shape(s1), ND.of_shape(s2)
        ref = np.zeros(c0.size, dtype=dt)
        oracle.broadcast(op, ref, c0.as_inline_array(), h, c1.as_inline_array(), dr, c2.as_inline_array(), d=d)
        got = gpu_call3(L.lib.nk_broadcast, device, L.OPS[op], np.zeros(c0.size, dtype=dt), c0, h, c1, dr, c2, d=d)
        if op in ("+", "-", "*"):
            assert np.array_equal(got, ref), f"{op} {s0} d={d}"
        else:
            np.testing.assert_allclose(got, ref, rtol=1e-5 if dt == np.float32 else 1e-12)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("op", OPS + ["idy"])
@pytest.mark.parametrize("d", [-1, 0, 1])
def test_scalar_broadcast(device, oracle, dt, op, d):
    rng = np.random.default_rng(37)
    c0, n0 = rand_view(rng, [6, 50], "sliced")
    c1, n1 = rand_view(rng, [6, 50], "dense")
    a = _inputs(rng, n1, dt, positive=(op == "**"))
    value = 1.75
    ref = np.zeros(n0, dtype=dt)
    oracle.scalar_broadcast(op, ref, c0.as_inline_array(), a, c1.as_inline_array(), value, d=d, threads=2)
    code = L.NK_OP_IDY if op == "idy" else L.OPS[op]
    got = gpu_scalar(device, code, np.zeros(n0, dtype=dt), c0, a, c1, value, d=d)
    _assert_close(got, ref, 1 if op in ("**", "/", "%") else 0, f"scalar {op} d={d}")


def test_fill_fun_sum_and_errors(device, oracle):
    for dt in (np.float32, np.float64):
        c0, n0 = rand_view(np.random.default_rng(41), [5, 9], "strided")
        D = DevArray(device, np.zeros(n0, dtype=dt))
        k, p = cfgp(c0)
        L.check(L.lib.nk_fill_fun(device.ctx, L.FUN["tanh"], D.nk_dtype, 2, D.buf, p, 0.3, -1), device.ctx)
        got = D.read()
        want = oracle.fun32("tanh", 0.3) if dt == np.float32 else oracle.fun64("tanh", 0.3)
        assert np.all(ulp_diff(got[c0.element_offsets()], np.full(c0.size, want, dtype=dt)) <= 1)
        mask = np.ones(n0, dtype=bool); mask[c0.element_offsets()] = False
        assert np.all(got[mask] == 0)
        # sum in CPUSum's tile order: bit-exact
        rng = np.random.default_rng(43)
        for n in (1, 5, 128, 129, 16384, 100_003):
            x = rng.standard_normal(n).astype(dt)
            S, O = DevArray(device, x), DevArray(device, np.zeros(2, dtype=dt))
            k, p = cfgp(ND.of_shape([n]))
            L.check(L.lib.nk_sum(device.ctx, S.nk_dtype, 1, S.buf, p, O.buf, 1), device.ctx)
            assert O.read()[1] == dt(oracle.cpu_sum(x)), n
    # unsupported dtype / mismatching shapes raise
    x = DevArray(device, np.zeros(4, dtype=np.float32))
    k, p = cfgp(ND.of_shape([4])); k3, p3 = cfgp(ND.of_shape([3]))
    assert L.lib.nk_unary(device.ctx, 0, L.NK_I32, 1, x.buf, p, x.buf, p, -1) == L.NK_ERR_UNSUPPORTED
    assert L.lib.nk_unary(device.ctx, 99, L.NK_F32, 1, x.buf, p, x.buf, p, -1) == L.NK_ERR_BAD_ARG
    assert L.lib.nk_binary(device.ctx, 0, L.NK_F32, 1, x.buf, p, x.buf, p3, x.buf, p, -1) == L.NK_ERR_BAD_ARG
    assert b"shapes differ" in L.lib.nk_last_error(device.ctx)


def test_large_broadcast_rows_kernel(device, oracle):
    """The shape family of the broadcast benchmark (a [n,1,k] * b [1,m,k]) at a size that takes the vectorised
    row kernel, checked exactly."""
    rng = np.random.default_rng(47)
    dt = np.float32
    a = (rng.random(64 * 1024, dtype=np.float32) * 4 - 2)
    b = (rng.random(48 * 1024, dtype=np.float32) * 4 - 2)
    c0, c1, c2 = ND.of_shape([64, 48, 1024]), ND.of_shape([64, 1, 1024]), ND.of_shape([1, 48, 1024])
    got = gpu_call3(L.lib.nk_broadcast, device, L.NK_OP_MUL, np.zeros(c0.size, dtype=dt), c0, a, c1, b, c2)
    assert device.last_kernel() == "nk_ew_rows_kernel"
    want = (a.reshape(64, 1, 1024) * b.reshape(1, 48, 1024)).reshape(-1)
    assert np.array_equal(got, want)


def test_permuted_slices_as_operands(device, oracle):
    """A permuted view of a strided slice (the reference's SimpleReshapeView) as operand of a broadcast, an activation
    and a convolution: the kernels only see its inline array, the oracle resolves the same array on the CPU."""
    from neureka_b200.tensor import Tensor
    from neureka_b200.functions import Function
    rng = np.random.default_rng(77)
    parent = Tensor.of(np.float32, [10, 12, 9], rng.uniform(-2, 2, 10 * 12 * 9).astype(np.float32)).to(device)
    view = parent[1:9:2, 2:12:2, 0:8].permute(2, 0, 1)          # [8, 4, 5]
    assert view.shape == (8, 4, 5)
    host = parent.numpy()[1:9:2, 2:12:2, 0:8].transpose(2, 0, 1)
    assert np.array_equal(view.numpy(), host)
    other = Tensor.of(np.float32, [8, 1, 5], rng.uniform(-2, 2, 40).astype(np.float32)).to(device)
    got = Function.of("tanh(i0 * i1) + i0", False)(view, other)
    h64 = host.astype(np.float32)
    t = (h64 * other.numpy()).astype(np.float32)
    want = np.array([oracle.fun32("tanh", float(v)) for v in t.reshape(-1)], dtype=np.float32).reshape(t.shape) + h64
    assert np.abs(got.numpy() - want).max() <= 2 * np.finfo(np.float32).eps * np.abs(want).max()
    k = Tensor.of(np.float32, [1, 3, 3], rng.standard_normal(9).astype(np.float32)).to(device)
    y = Function.of("i0 x i1", False)(view, k)
    ref = np.zeros((8, 2, 3), dtype=np.float32)
    for c in range(8):
        for i in range(2):
            for j in range(3):
                ref[c, i, j] = np.sum(host[c, i:i + 3, j:j + 3].astype(np.float64) * k.numpy()[0].astype(np.float64))
    assert np.abs(y.numpy() - ref).max() <= 1e-5 * np.abs(ref).max() * 4
