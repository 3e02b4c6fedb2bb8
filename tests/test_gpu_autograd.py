"""The reference's end-to-end known answers for the path, run through the Function layer on the CUDA device:
Function.of("i0 x i1"), XConvLeft/XConvRight, backward() of convolutions, broadcasting + / - / *, tanh."""
import numpy as np
import pytest

from neureka_b200 import _lib as L
from neureka_b200.functions import Function
from neureka_b200.tensor import Tensor

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_conv_operator_golden(device, kat, dt):
    for v in kat["conv_forward"]:
        x = Tensor.of(dt, v["a_shape"], v["a"]).to(device)
        k = Tensor.of(dt, v["b_shape"], v["b"]).to(device)
        y = x.conv(k)
        assert y.shape == tuple(v["out_shape"]) and y.items.tolist() == [float(t) for t in v["out"]], v["src"]
        z = Function.of("I0xi1")(x, k)
        assert z.items.tolist() == [float(t) for t in v["out"]]


def test_host_operand_is_stored_for_the_call_and_restored(device):
    x = Tensor.of(np.float64, [3, 3], np.arange(1, 10)).to(device)
    k = Tensor.of(np.float64, [2, 2], [1, 2, 0, -1])          # stays on the host
    y = Function.of("i0 x i1")(x, k)
    assert y.items.tolist() == [0, 2, 6, 8]
    assert not k.is_outsourced and device.has(y)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_xconv_operators(device, kat, dt):
    v = kat["xconv"][0]
    t1 = Tensor.of(dt, v["drain_shape"], [0] * 6).to(device)
    t2 = Tensor.of(dt, v["t1_shape"], v["t1"]).to(device)
    t3 = Tensor.of(dt, v["t2_shape"], v["t2"]).to(device)
    r = Function.of("i0<<xi1<<xi2")(t1, t2, t3)
    assert r.items.tolist() == [float(x) for x in v["out"]]
    t1 = Tensor.of(dt, v["drain_shape"], [0] * 6).to(device)
    r = Function.of("i2x>>i1x>>i0")(t1, t2, t3)
    assert r.items.tolist() == [float(x) for x in v["out"]]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_conv_backward_golden(device, kat, dt):
    for v in kat["conv_autograd"]:
        a = Tensor.of(dt, v["a_shape"], v["a"]).set_rqs_gradient(True).to(device)
        b = Tensor.of(dt, v["b_shape"], v["b"]).to(device)
        z = Function.of("i0xi1")(a, b)
        z.backward(Tensor.of(dt, v["error_shape"], v["error"]))
        assert a.gradient.items.tolist() == [float(x) for x in v["grad_a"]], v["src"]


def test_two_layer_convolution_chain(device, kat):
    v = kat["conv_autograd_chain"]
    dt = np.float64
    i_a = Tensor.of(dt, v["i_a"]["shape"], v["i_a"]["data"]).to(device)
    w_a = Tensor.of(dt, v["w_a"]["shape"], v["w_a"]["data"]).set_rqs_gradient(True).to(device)
    w_b = Tensor.of(dt, v["w_b"]["shape"], v["w_b"]["data"]).set_rqs_gradient(True).to(device)
    w_c = Tensor.of(dt, v["w_c"]["shape"], v["w_c"]["data"]).set_rqs_gradient(True).to(device)
    conv = Function.of("i0 x i1")
    o_a = conv(i_a, w_a)
    o_b, o_c = conv(o_a, w_b), conv(o_a, w_c)
    out = o_b * o_c
    assert o_a.items.tolist() == v["o_a"] and o_b.items.tolist() == v["o_b"] and o_c.items.tolist() == v["o_c"]
    assert out.items.tolist() == v["out"]
    out.backward(Tensor.of(dt, [2, 1], 1.0))
    assert w_b.gradient.items.tolist() == v["grad_w_b"]
    assert (w_a.items + w_a.gradient.items).tolist() == v["w_a_after_apply"]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_broadcast_autograd_table(device, kat, dt):
    ops = {"+": lambda x, y: x + y, "-": lambda x, y: x - y, "*": lambda x, y: x * y, "rsub": lambda x, y: y - x}
    for row in kat["broadcast_autograd"]:
        wb = row["which_grad"] == "b"
        a = Tensor.of(dt, [2, 2], [1, 2, 3, 4]).set_rqs_gradient(not wb).to(device)
        b = Tensor.of(dt, row["b_shape"], [8, 9]).set_rqs_gradient(wb).to(device)
        c = ops[row["op"]](a, b)
        assert c.items.tolist() == [float(x) for x in row["c"]], row["src"]
        c.backward(Tensor.of(dt, [2, 2], [5, -2, 7, 3]))
        w = b if wb else a
        assert w.gradient.shape == w.shape
        assert w.gradient.items.tolist() == [float(x) for x in row["grad"]], row["src"]


def test_tanh_chain_golden(device, kat):
    v = kat["tanh_chain"]
    x = Tensor.of(np.float64, [1], [v["x"]]).set_rqs_gradient(True).to(device)
    z = Function.of("i0*100")(Function.of("tanh(i0)")(x))
    assert round(float(z.item()), 4) == v["value_4dp"]
    z.backward(Tensor.of(np.float64, [1], [1.0]))
    assert round(float(x.gradient.item()), 4) == v["grad_4dp"]


def test_scaled_config3_forward_and_reduced_gradients(device, oracle):
    """BASELINE config 3 at a reduced size: y = tanh(i0*i1+i1) with a [n,1,k], b [1,m,k]; backward of sum(y).
    Forward is checked against the oracle op by op (<= 1 ulp per op => compare the final result to the oracle's
    own chain); the gradients are the mathematically reduced ones: da = sum_j g*b, db = sum_i g*(a+1)."""
    import ctypes as C
    from neureka_b200 import _lib as L
    from neureka_b200.ndconf import NDConfiguration as ND
    n, m, k = 24, 16, 160
    dt = np.float32
    import baseline_configs as B
    a_h, b_h = B.cfg3_inputs(n, m, k)   # one uniform stream of seed 3: a, then b
    a = Tensor.of(dt, [n, 1, k], a_h).set_rqs_gradient(True).to(device)
    b = Tensor.of(dt, [1, m, k], b_h).set_rqs_gradient(True).to(device)
    y = Function.of("tanh(i0*i1+i1)")(a, b)
    # oracle chain
    co, ca, cb = ND.of_shape([n, m, k]), ND.of_shape([n, 1, k]), ND.of_shape([1, m, k])
    t1, t2, ref = (np.zeros(co.size, dtype=dt) for _ in range(3))
    oracle.broadcast("*", t1, co.as_inline_array(), a_h, ca.as_inline_array(), b_h, cb.as_inline_array())
    oracle.broadcast("+", t2, co.as_inline_array(), t1, co.as_inline_array(), b_h, cb.as_inline_array())
    oracle.unary("tanh", ref, co.as_inline_array(), t2, co.as_inline_array())
    from helpers import ulp_diff
    assert ulp_diff(y.items, ref).max() <= 1
    s = y.sum()
    assert float(s.item()) == pytest.approx(float(oracle.cpu_sum(y.items)), rel=1e-6)
    s.backward()
    g = np.zeros(co.size, dtype=dt)
    oracle.unary("tanh", g, co.as_inline_array(), t2, co.as_inline_array(), d=0)
    g3 = g.reshape(n, m, k).astype(np.float64)
    da = (g3 * b_h.reshape(1, m, k)).sum(axis=1)
    db = (g3 * (a_h.reshape(n, 1, k).astype(np.float64) + 1)).sum(axis=0)
    np.testing.assert_allclose(a.gradient.items.reshape(n, k), da, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(b.gradient.items.reshape(m, k), db, rtol=1e-5, atol=1e-5)


def test_config3_through_the_api_at_the_largest_int_sized_variant(device, oracle):
    """BASELINE config 3 through Function.of("tanh(i0*i1+i1)") and backward(), at 2^30 outputs: a [1024,1,1024],
    b [1,1024,1024] -- the largest variant of the configuration whose tensors a Java int can still count (the full
    2^33 cannot exist in the reference). Same generator and seed as the full size. Forward: sampled windows against
    the oracle's op-by-op chain, <= 1 ulp. Backward of the sum: rows of the reduced gradients against float64 sums."""
    import baseline_configs as B
    from helpers import ulp_diff
    from neureka_b200.ndconf import NDConfiguration as ND
    if device.props.total_mem_bytes < 60 * (1 << 30):
        pytest.skip("needs ~40 GiB of device memory")
    n, m, k = 1024, 1024, 1024
    dt = np.float32
    a_h, b_h = B.cfg3_inputs(n, m, k)
    a = Tensor.of(dt, [n, 1, k], a_h).set_rqs_gradient(True).to(device)
    b = Tensor.of(dt, [1, m, k], b_h).set_rqs_gradient(True).to(device)
    y = Function.of("tanh(i0*i1+i1)")(a, b)
    assert y.shape == (n, m, k) and y.is_outsourced
    N = n * m * k
    win = 8192
    rng = np.random.default_rng(31)
    acc = device.access(y)
    cw = ND.of_shape([win]).as_inline_array()
    for s0 in [0, N - win, (1 << 29) - 17] + [int(x) for x in rng.integers(0, N - win, size=8)]:
        got = acc.read_array(s0, win)
        idx = np.arange(s0, s0 + win, dtype=np.int64)
        i, j, kk = idx // (m * k), (idx // k) % m, idx % k
        av, bv = a_h[i * k + kk], b_h[j * k + kk]
        t1, t2, want = (np.zeros(win, dtype=dt) for _ in range(3))
        oracle.bielementwise("*", t1, cw, np.ascontiguousarray(av), cw, np.ascontiguousarray(bv), cw)
        oracle.bielementwise("+", t2, cw, t1, cw, np.ascontiguousarray(bv), cw)
        oracle.unary("tanh", want, cw, t2, cw)
        assert ulp_diff(got, want).max() <= 1, s0
    s = y.sum()
    s.backward()
    ga = a.gradient.items.reshape(n, k)
    gb = b.gradient.items.reshape(m, k)
    A, Bm = a_h.reshape(n, k), b_h.reshape(m, k)

    def g_of(arow, brow):   # tanh'(a*b+b) as the reference defines it for F32, evaluated in float64
        u = (arow * brow).astype(np.float32) + brow
        t = np.zeros(u.size, dtype=np.float32)
        c = ND.of_shape([u.size]).as_inline_array()
        oracle.unary("tanh", t, c, np.ascontiguousarray(u.reshape(-1)), c, d=0)
        return t.reshape(u.shape).astype(np.float64)

    for i in (0, 511, n - 1):      # da[i, :] = sum_j g[i, j, :] * b[j, :]
        g = g_of(A[i][None, :], Bm)
        want = (g * Bm).sum(axis=0)
        mag = (np.abs(g) * np.abs(Bm)).sum(axis=0)
        assert np.all(np.abs(ga[i] - want) <= 1e-5 * mag + 1e-30)
    for j in (0, 300, m - 1):      # db[j, :] = sum_i g[i, j, :] * (a[i, :] + 1)
        g = g_of(A, Bm[j][None, :])
        want = (g * (A.astype(np.float64) + 1)).sum(axis=0)
        mag = (np.abs(g) * (np.abs(A.astype(np.float64)) + 1)).sum(axis=0)
        assert np.all(np.abs(gb[j] - want) <= 1e-5 * mag + 1e-30)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("mkn", [(3, 4, 2), (70, 130, 50), (256, 192, 160)])
def test_matmul_operator_forward_and_backward(device, dt, mkn):
    """`@` (linear/MatMul.java, algorithms/MatMulAlgorithm.java:37-59) on the convolution kernels: forward against numpy in
    float64, the gradients of sum(a @ b * w) against their closed forms; the largest case takes the contraction kernel."""
    m, k, n = mkn
    rng = np.random.default_rng(m * 1000 + n)
    a_h, b_h, w_h = rng.standard_normal((m, k)), rng.standard_normal((k, n)), rng.standard_normal((m, n))
    a = Tensor.of(dt, [m, k], a_h).set_rqs_gradient(True).to(device)
    b = Tensor.of(dt, [k, n], b_h).set_rqs_gradient(True).to(device)
    c = Function.of("i0 @ i1")(a, b)
    tol = (1e-5 if dt == np.float32 else 1e-12) * k * 4
    ref = a_h.astype(dt).astype(np.float64) @ b_h.astype(dt).astype(np.float64)
    assert c.shape == (m, n)
    assert np.abs(c.numpy() - ref).max() <= tol * max(1.0, np.abs(ref).max()) / k
    if m * k * n >= (1 << 21):
        from neureka_b200 import _lib as L
        assert device.last_conv_path() in (L.NK_CONV_GEMM, L.NK_CONV_TC)
    c.backward(Tensor.of(dt, [m, n], w_h))
    ga = w_h.astype(dt).astype(np.float64) @ b_h.astype(dt).astype(np.float64).T
    gb = a_h.astype(dt).astype(np.float64).T @ w_h.astype(dt).astype(np.float64)
    assert np.abs(a.gradient.numpy() - ga).max() <= tol * max(1.0, np.abs(ga).max())
    assert np.abs(b.gradient.numpy() - gb).max() <= tol * max(1.0, np.abs(gb).max())
    # the operator form and a transposed view as operand
    c2 = a @ b
    assert np.array_equal(c2.numpy(), c.numpy())
    c3 = Function.of("i0 @ i1", False)(b.T, a.T)
    assert np.abs(c3.numpy() - ref.T).max() <= tol * max(1.0, np.abs(ref).max()) / k
    with pytest.raises(ValueError):
        Function.of("i0 @ i1", False)(a, a)


def test_dot_product_golden_vectors_and_autograd(device, kat, oracle):
    """Tensor_Dot_Product_Spec.groovy: forward values, the gradient of the weight vector for error 0.5, and a long pair of
    vectors against the oracle's restatement of CPUDot (DOT.unrolled04's four partial sums)."""
    for v in kat["dot"]:
        for dt in (np.float32, np.float64):
            a = Tensor.of(dt, [len(v["a"])], v["a"]).to(device)
            b = Tensor.of(dt, [len(v["b"])], v["b"]).set_rqs_gradient("grad_b" in v).to(device)
            r = a.dot(b)
            assert r.shape == (1,) and r.items.tolist() == [v["value"]]
            assert oracle.dot(np.asarray(v["a"], dtype=dt), np.asarray(v["b"], dtype=dt)) == v["value"]
            if "grad_b" in v:
                r.backward(Tensor.of(dt, [1], [v["error"]]))
                assert b.gradient.items.tolist() == v["grad_b"]
    rng = np.random.default_rng(3)
    n = 300_001
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    got = float(Tensor.of(np.float32, [n], x).to(device).dot(Tensor.of(np.float32, [n], y).to(device)).item())
    want = oracle.dot(x, y)
    assert abs(got - want) <= 1e-5 * float(np.abs(x.astype(np.float64) * y).sum())
    with pytest.raises(ValueError, match="vectors"):
        Tensor.of(np.float32, [2, 2], [1, 2, 3, 4]).to(device).dot(Tensor.of(np.float32, [2, 2], [1, 2, 3, 4]).to(device))
    with pytest.raises(ValueError, match="same length"):
        Tensor.of(np.float32, [2], [1, 2]).to(device).dot(Tensor.of(np.float32, [3], [1, 2, 3]).to(device))


def test_matmul_golden_vectors_and_oracle(device, kat, oracle):
    """Matrix_Multiplication_Spec.groovy's vectors through `@`, and larger products against the oracle's restatement of
    CPUMatMul (GEMM.partial_F32_MxN_RM: products added in rising order of the common index) within 1e-5 / 1e-12 of
    sum|a||b| per element -- through the FMA contraction family and, for the largest, the tensor cores."""
    for v in kat["matmul"]:
        for dt in (np.float32, np.float64):
            a = Tensor.of(dt, [v["M"], v["K"]], v["a"]).to(device)
            b = Tensor.of(dt, [v["K"], v["N"]], v["b"]).to(device)
            c = a @ b
            assert c.shape == (v["M"], v["N"]) and c.items.tolist() == v["c"]
            ref = oracle.matmul(np.asarray(v["a"], dtype=dt).reshape(v["M"], v["K"]), np.asarray(v["b"], dtype=dt).reshape(v["K"], v["N"]))
            assert ref.reshape(-1).tolist() == v["c"]
    rng = np.random.default_rng(8)
    for dt, tol, (m, k, n) in ((np.float32, 1e-5, (96, 130, 80)), (np.float64, 1e-12, (96, 130, 80)), (np.float32, 1e-5, (384, 512, 320))):
        a_h, b_h = rng.standard_normal((m, k)).astype(dt), rng.standard_normal((k, n)).astype(dt)
        c = Tensor.of(dt, [m, k], a_h).to(device) @ Tensor.of(dt, [k, n], b_h).to(device)
        ref = oracle.matmul(a_h, b_h)
        mag = np.abs(a_h).astype(np.float64) @ np.abs(b_h).astype(np.float64)
        assert np.all(np.abs(c.numpy().astype(np.float64) - ref) <= tol * mag)
    assert device.last_conv_path() == L.NK_CONV_TC


def test_min_and_max_return_the_extreme_item_and_route_the_error_to_its_index(device):
    """operations/other/Min.java / Max.java on CPUReduce's semantics: the first of equal extremes wins; backward puts the
    error at that index of a zero tensor."""
    rng = np.random.default_rng(12)
    for dt in (np.float32, np.float64):
        for shape in ([7], [65, 3], [1000, 333]):
            h = rng.standard_normal(int(np.prod(shape))).astype(dt)
            h[h.size // 3] = h[h.size // 2] = h.max() + 1      # two equal maxima: the earlier one is the answer
            h[5 % h.size] = h[h.size - 1] = h.min() - 1        # ... and two equal minima
            t = Tensor.of(dt, shape, h).set_rqs_gradient(True).to(device)
            mx, mn = t.max(), t.min()
            assert mx.shape == (1,) and float(mx.item()) == h.max() and float(mn.item()) == h.min()
            mx.backward(Tensor.of(dt, [1], [2.5]))
            g = t.gradient.items
            assert g[int(np.argmax(h))] == 2.5 and np.count_nonzero(g) == 1
    # a strided slice: the index counts the view's elements, the value is read through the view
    base = Tensor.of(np.float32, [6, 8], np.arange(48)).to(device)
    v = base[1:5:2, 2:8:3]            # rows 1, 3; columns 2, 5 -> items 10, 13, 26, 29
    assert float(v.max().item()) == 29 and float(v.min().item()) == 10
    import ctypes as C
    out = Tensor.of(np.float32, [1], [0]).to(device)     # a result buffer of the wrong type is refused
    k = base.ndconf.as_inline_array()
    st = L.lib.nk_arg_reduce(device.ctx, 1, L.NK_F32, 2, base._data.buf, k.ctypes.data_as(C.POINTER(C.c_int32)), out._data.buf, 0)
    assert st == L.NK_ERR_BAD_ARG
