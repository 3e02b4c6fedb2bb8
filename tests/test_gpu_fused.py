"""Fused elementwise expressions (CudaDevice.optimized_operation_of / nk_fused_*): one run-time compiled kernel per
Function must give exactly the bits of the op-by-op evaluation the reference performs (every operator rounds to the
tensor's type; the scalar functions are the same source), with broadcasting, on views, for F32 and F64."""
import ctypes as C

import numpy as np
import pytest

from neureka_b200 import _lib as L
from neureka_b200.functions import Function
from neureka_b200.tensor import Tensor

pytestmark = pytest.mark.gpu


def _bits(a):
    a = np.ascontiguousarray(a)
    return a.view(np.int32 if a.dtype == np.float32 else np.int64)


def _same_bits(a, b):
    # NaNs of different payloads are both "the NaN the formula produces"
    a, b = np.asarray(a), np.asarray(b)
    both_nan = np.isnan(a) & np.isnan(b)
    return bool(np.all((_bits(a) == _bits(b)) | both_nan))


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("expr,shapes", [
    ("tanh(i0*i1+i1)", [[64, 1, 96], [1, 48, 96]]),                      # BASELINE config 3 in small
    ("relu(i0) ** 2 - i1 / 3 % i2", [[40, 52], [40, 52], [40, 52]]),     # constants, all six operators but +
    ("-i0 + gaus(i1) * softplus(i2)", [[7, 1, 33], [1, 5, 33], [7, 5, 1]]),   # three-way broadcast, odd inner extent
    ("sig(silu(gelu(i0)))", [[1000]]),
    ("cbrt(i0) + sqrt(abs(i1)) + ln(quad(i1) + 1)", [[3, 4, 5, 6], [1, 4, 1, 6]]),
    ("fast_tanh(i0) * fast_gaus(i0) + selu(i0) - softsign(i0) + log10(abs(i0) + 2) + sin(cos(exp(i0 / 8)))", [[513]]),
])
def test_fused_equals_op_by_op_bit_for_bit(device, dt, expr, shapes):
    rng = np.random.default_rng(41)
    hosts = [rng.uniform(-2.0, 2.0, size=int(np.prod(s))).astype(dt) for s in shapes]
    tensors = [Tensor.of(dt, s, h).to(device) for s, h in zip(shapes, hosts)]
    f = Function.of(expr, False)
    want = f(*tensors)
    fused = device.optimized_operation_of(f, "fused_test")
    before = device.launch_count()
    got = fused(*tensors)
    assert device.launch_count() - before == 1 and device.last_kernel() in ("nk_fused_kernel", "nk_fused_rows_kernel")
    assert got.shape == want.shape
    assert _same_bits(got.items, want.items), np.abs(got.items - want.items).max()
    fused.close()


def test_fused_tanh_on_tiny_inputs_zeros_infinities_and_nans(device):
    """The F32 tanh has a straight-line form for ordinary inputs and the literal formula for |x| < 2^-26 and NaN; the fused
    kernel evaluates a vector with the first and repeats it with the second when an element asks for it. Vectors that mix
    both kinds must give the operator kernel's bits."""
    special = np.asarray([0.0, -0.0, 1e-9, -1e-9, 1.4e-45, 3e-39, 1.4901161e-08, 1.49e-08, np.inf, -np.inf, np.nan, 1e-20,
                          0.5, -0.5, 20.0, -20.5, 88.0, 1e30, -1e30, 2.0 ** -27], dtype=np.float32)
    rng = np.random.default_rng(5)
    x = rng.uniform(-3, 3, 4096).astype(np.float32)
    x[rng.choice(4096, 400, replace=False)] = rng.choice(special, 400)
    t = Tensor.of(np.float32, [16, 256], x).to(device)
    one = Tensor.of(np.float32, [1, 256], np.ones(256, dtype=np.float32)).to(device)
    f = Function.of("tanh(i0*i1)", False)
    fused = device.optimized_operation_of(f, "tanh_special")
    got, want = fused(t, one), f(t, one)
    assert _same_bits(got.items, want.items)
    fused.close()


def test_fused_on_views_and_against_the_oracle(device, oracle):
    """A strided slice and a permuted operand; and the fused tanh(a*b+b) against the CPU restatement (<= 1 ulp)."""
    rng = np.random.default_rng(42)
    a_parent = Tensor.of(np.float32, [20, 64], rng.uniform(-2, 2, 20 * 64).astype(np.float32)).to(device)
    a = a_parent[2:18:2, 0:64]                       # [8, 64], every second row
    b_t = Tensor.of(np.float32, [64, 8], rng.uniform(-2, 2, 64 * 8).astype(np.float32)).to(device)
    b = b_t.permute(1, 0)                            # [8, 64] column-major view
    f = Function.of("tanh(i0*i1+i1)", False)
    fused = device.optimized_operation_of(f, "tanh_affine")
    got = fused(a, b)
    want = f(a, b)
    assert _same_bits(got.items, want.items)
    an, bn = a.numpy().astype(np.float32), b.numpy().astype(np.float32)
    u = (an * bn).astype(np.float32) + bn
    ref = np.array([oracle.fun32("tanh", float(v)) for v in u.reshape(-1)], dtype=np.float32)
    d = np.abs(_bits(got.items.astype(np.float32)).astype(np.int64) - _bits(ref).astype(np.int64))
    assert d.max() <= 1
    fused.close()


def test_fused_config3_scaled(device):
    """a [1024,1,1024], b [1,1024,1024] -> 2^30 outputs in one pass; equals the three-kernel evaluation."""
    rng = np.random.default_rng(43)
    n = 1024
    a = Tensor.of(np.float32, [n, 1, n], rng.uniform(-2, 2, n * n).astype(np.float32)).to(device)
    b = Tensor.of(np.float32, [1, n, n], rng.uniform(-2, 2, n * n).astype(np.float32)).to(device)
    f = Function.of("tanh(i0*i1+i1)", False)
    fused = device.optimized_operation_of(f, "cfg3")
    got = fused(a, b)
    want = f(a, b)
    # compare on the device side of things cheaply: windows of the 4 GiB results
    for start in (0, n * n * 511 + 77, n * n * n - 4096):
        g = device.access(got).read_array(start, 4096)
        w = device.access(want).read_array(start, 4096)
        assert _same_bits(g, w)
    fused.close()


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("expr,shapes", [
    ("tanh(i0*i1+i1)", [[64, 1, 96], [1, 48, 96]]),                      # BASELINE config 3 in small: b occurs twice
    ("i0*i1 - i2", [[5, 1, 32], [1, 7, 32], [5, 7, 1]]),                 # the innermost dim is summed away for i2
    ("relu(i0) + sig(i0) * i1", [[40, 52], [40, 52]]),                    # no broadcasting: nothing to reduce
    ("sin(i0) * i1", [[33, 20], [1, 1]]),                                 # a single element against a matrix
])
def test_fused_backward_equals_op_by_op_bit_for_bit(device, dt, expr, shapes):
    """backward() through a fused operation: per input one kernel that multiplies the error through the expression and
    sums over the dims that input is broadcast along. Every product rounds like the op-by-op pass, every occurrence of an
    input is summed separately in the reduction kernels' order, and these expressions reduce at one node each: the
    gradients equal the op-by-op gradients bit for bit. The forward result is checked on the way."""
    rng = np.random.default_rng(47)
    hosts = [rng.uniform(-2.0, 2.0, size=int(np.prod(s))).astype(dt) for s in shapes]
    out_shape = [max(s[k] for s in shapes) for k in range(len(shapes[0]))]
    err_h = rng.uniform(-1.0, 1.0, size=int(np.prod(out_shape))).astype(dt)

    def run(make_result):
        ts = [Tensor.of(dt, s, h).set_rqs_gradient(True).to(device) for s, h in zip(shapes, hosts)]
        y = make_result(ts)
        y.backward(Tensor.of(dt, out_shape, err_h))
        return y.items, [t.gradient.items for t in ts]

    f = Function.of(expr)
    fused = device.optimized_operation_of(f, "fused_backward_test")
    y_ref, g_ref = run(lambda ts: f(*ts))
    n0 = device.launch_count()
    y_fus, g_fus = run(lambda ts: fused(*ts))
    assert _same_bits(y_fus, y_ref)
    for j, (a, b) in enumerate(zip(g_fus, g_ref)):
        assert a.shape == b.shape
        assert _same_bits(a, b), (j, np.abs(a - b).max())
    fused.close()


def test_fused_backward_of_a_sum_takes_one_kernel_per_input(device, oracle):
    """sum(tanh(a*b+b)).backward() with a [n,1,k], b [1,m,k] through the fused operation: the virtual all-ones error stays
    one element, each gradient is one launch of the gradient kernel, and no result-sized tensor besides the forward
    result exists. Checked against float64 sums of the oracle's tanh derivative."""
    from neureka_b200.ndconf import NDConfiguration as ND
    import baseline_configs as BC
    n, m, k = 48, 40, 256
    a_h, b_h = BC.cfg3_inputs(n, m, k)
    a = Tensor.of(np.float32, [n, 1, k], a_h).set_rqs_gradient(True).to(device)
    b = Tensor.of(np.float32, [1, m, k], b_h).set_rqs_gradient(True).to(device)
    fused = device.optimized_operation_of(Function.of("tanh(i0*i1+i1)"), "cfg3")
    y = fused(a, b)
    s = y.sum()
    n0 = device.launch_count()
    s.backward()
    kernels = device.launch_count() - n0
    assert device.last_kernel() != "" and kernels <= 8, kernels     # two gradient kernels + the assigns into .gradient
    A, Bm = a_h.reshape(n, 1, k).astype(np.float32), b_h.reshape(1, m, k).astype(np.float32)
    u = (A * Bm).astype(np.float32) + Bm
    g = np.zeros(u.size, dtype=np.float32)
    c = ND.of_shape([u.size]).as_inline_array()
    oracle.unary("tanh", g, c, np.ascontiguousarray(u.reshape(-1)), c, d=0)
    g = g.reshape(n, m, k).astype(np.float64)
    da = (g * Bm).sum(axis=1)
    db = (g * (A.astype(np.float64) + 1)).sum(axis=0)
    mag_a = (np.abs(g) * np.abs(Bm)).sum(axis=1)
    mag_b = (np.abs(g) * (np.abs(A) + 1)).sum(axis=0)
    assert np.all(np.abs(a.gradient.items.reshape(n, k) - da) <= 1e-5 * mag_a + 1e-30)
    assert np.all(np.abs(b.gradient.items.reshape(m, k) - db) <= 1e-5 * mag_b + 1e-30)
    fused.close()


def test_fused_refuses_what_it_cannot_do(device):
    with pytest.raises(ValueError, match="not elementwise"):
        device.optimized_operation_of(Function.of("i0 x i1", False), "conv")
    a = Tensor.of(np.float32, [4, 5], np.ones(20)).to(device)
    b = Tensor.of(np.float32, [3, 5], np.ones(15)).to(device)
    fused = device.optimized_operation_of(Function.of("i0 + i1", False), "add")
    with pytest.raises(ValueError, match="broadcast"):
        fused(a, b)
    with pytest.raises(ValueError, match="takes 2 inputs"):
        fused(a)
    # a malformed expression reaches the caller with the compiler's message
    h = C.c_void_p()
    st = L.lib.nk_fused_compile(device.ctx, L.NK_F32, 1, b"f_no_such_function(x0)", C.byref(h))
    assert st == L.NK_ERR_BAD_ARG and b"f_no_such_function" in L.lib.nk_last_error(device.ctx)
    assert L.lib.nk_fused_compile(device.ctx, L.NK_I32, 1, b"x0", C.byref(h)) == L.NK_ERR_UNSUPPORTED
    assert L.lib.nk_fused_compile(device.ctx, L.NK_F32, 9, b"x0", C.byref(h)) == L.NK_ERR_BAD_ARG
    assert L.lib.nk_fused_free(None) == L.NK_ERR_BAD_ARG
