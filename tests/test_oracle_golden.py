"""Pins the CPU oracle (oracle/oracle.cpp) against the known-answer vectors transcribed from the reference's
own tests (tests/golden/reference_kat.json): only an oracle that reproduces them may be used to check the CUDA path."""
import numpy as np
import pytest

from neureka_b200.ndconf import Layout, NDConfiguration as ND

DTYPES = [np.float32, np.float64]


def _conv(O, dt, sa, a, sb, b, so, ca=None, cb=None, threads=1, allow_simple=True, d=-1):
    A, Bv = np.asarray(a, dtype=dt), np.asarray(b, dtype=dt)
    out = np.zeros(int(np.prod(so)), dtype=dt)
    ca = ca or ND.of_shape(sa)
    cb = cb or ND.of_shape(sb)
    O.conv(out, ND.of_shape(so).as_inline_array(), A, ca.as_inline_array(), Bv, cb.as_inline_array(), d=d, threads=threads, allow_simple=allow_simple)
    return out


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("threads", [1, 3])
@pytest.mark.parametrize("allow_simple", [True, False])
def test_forward_conv_vectors(oracle, kat, dt, threads, allow_simple):
    for v in kat["conv_forward"]:
        out = _conv(oracle, dt, v["a_shape"], v["a"], v["b_shape"], v["b"], v["out_shape"], threads=threads, allow_simple=allow_simple)
        assert out.tolist() == [float(x) for x in v["out"]], v["src"]


@pytest.mark.parametrize("dt", DTYPES)
def test_forward_conv_constant_matrix_product(oracle, kat, dt):
    v = kat["conv_forward_constant"][0]
    a = np.full(int(np.prod(v["a_shape"])), v["a_fill"], dtype=dt)
    b = np.full(int(np.prod(v["b_shape"])), v["b_fill"], dtype=dt)
    out = _conv(oracle, dt, v["a_shape"], a, v["b_shape"], b, v["out_shape"], threads=4)
    assert np.all(out == v["out_fill"])


def test_column_major_operands_give_the_same_result(oracle, kat):
    v = kat["conv_forward_column_major"][0]
    cb = ND.of_shape(v["b_shape"], Layout.COLUMN_MAJOR)
    assert cb.layout() is Layout.COLUMN_MAJOR
    # the raw data array of the column-major tensor is the permuted one the reference test lists
    raw = np.zeros(6)
    raw[cb.element_offsets()] = v["b"]
    assert raw.tolist() == [float(x) for x in v["b_raw_column_major"]]
    ca = ND.of_shape(v["a_shape"], Layout.COLUMN_MAJOR)
    a_raw = np.zeros(6)
    a_raw[ca.element_offsets()] = v["a"]
    out = _conv(oracle, np.float64, v["a_shape"], a_raw, v["b_shape"], raw, v["out_shape"], ca=ca, cb=cb)
    assert out.tolist() == [float(x) for x in v["out"]]


def test_conv_on_strided_slice(oracle, kat):
    v = kat["conv_forward_sliced"][0]
    parent = ND.of_shape(v["parent_shape"])
    sl = parent.sliced(v["slice_shape"], v["slice_offset"], v["slice_spread"])
    data = np.asarray(v["parent"], dtype=np.float64)
    assert data[sl.element_offsets()].tolist() == [float(x) for x in v["slice_items"]]
    out = _conv(oracle, np.float64, v["slice_shape"], data, v["b_shape"], v["b"], [1, 1], ca=sl)
    assert out.tolist() == [float(x) for x in v["out"]]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("threads", [1, 4])
def test_xconv_vector(oracle, kat, dt, threads):
    v = kat["xconv"][0]
    out = _conv(oracle, dt, v["t1_shape"], v["t1"], v["t2_shape"], v["t2"], v["drain_shape"], d=0, threads=threads)
    assert out.tolist() == [float(x) for x in v["out"]]


@pytest.mark.parametrize("dt", DTYPES)
def test_conv_autograd_vectors_via_deconvolution(oracle, kat, dt):
    # grad_a = XConvRight(error, b, zeros(a.shape)) -> implementation sees (zeros, b, error) with d = 0
    for v in kat["conv_autograd"]:
        rank = max(len(v["a_shape"]), len(v["b_shape"]))
        g = _conv(oracle, dt, v["b_shape"], v["b"], v["error_shape"], v["error"], v["a_shape"], d=0)
        assert g.tolist() == [float(x) for x in v["grad_a"]], v["src"]
        assert rank == len(v["error_shape"])


def test_two_layer_conv_chain(oracle, kat):
    v = kat["conv_autograd_chain"]
    dt = np.float64
    i_a, w_a, w_b, w_c = (np.asarray(v[k]["data"], dtype=dt) for k in ("i_a", "w_a", "w_b", "w_c"))
    o_a = _conv(oracle, dt, [2, 1], i_a, [2, 2], w_a, [1, 2])
    assert o_a.tolist() == v["o_a"]
    o_b = _conv(oracle, dt, [1, 2], o_a, [2, 2], w_b, [2, 1])
    o_c = _conv(oracle, dt, [1, 2], o_a, [2, 2], w_c, [2, 1])
    assert o_b.tolist() == v["o_b"] and o_c.tolist() == v["o_c"]
    assert (o_b * o_c).tolist() == v["out"]
    # d out / d o_b = o_c (error ones) ; grad w_b = XConvRight(err_b, o_a, zeros[2,2]) -> (zeros, o_a, err_b)
    g_wb = _conv(oracle, dt, [1, 2], o_a, [2, 1], o_c, [2, 2], d=0)
    assert g_wb.tolist() == v["grad_w_b"]
    # grad o_a = deconv(zeros[1,2], w_b, err_b) + deconv(zeros[1,2], w_c, err_c); grad w_a = deconv(zeros[2,2], i_a, grad o_a)
    g_oa = _conv(oracle, dt, [2, 2], w_b, [2, 1], o_c, [1, 2], d=0) + _conv(oracle, dt, [2, 2], w_c, [2, 1], o_b, [1, 2], d=0)
    g_wa = _conv(oracle, dt, [2, 1], i_a, [1, 2], g_oa, [2, 2], d=0)
    assert (w_a + g_wa).tolist() == v["w_a_after_apply"]


@pytest.mark.parametrize("dt", DTYPES)
def test_broadcast_forward_and_backward(oracle, kat, dt):
    v = kat["broadcast_forward_mul"][0]
    out = np.zeros(6, dtype=dt)
    oracle.broadcast("*", out, ND.of_shape(v["out_shape"]).as_inline_array(), np.asarray(v["a"], dtype=dt), ND.of_shape(v["a_shape"]).as_inline_array(),
                     np.asarray(v["b"], dtype=dt), ND.of_shape(v["b_shape"]).as_inline_array())
    assert out.tolist() == [float(x) for x in v["out"]]
    w = kat["broadcast_backward_mul_both"][0]
    origin = np.zeros(3, dtype=dt)
    oracle.broadcast("test_mul", origin, ND.of_shape(w["origin_shape"]).as_inline_array(), np.asarray(w["handle"], dtype=dt),
                     ND.of_shape(w["handle_shape"]).as_inline_array(), np.asarray(w["drain"], dtype=dt), ND.of_shape(w["drain_shape"]).as_inline_array(), d=0, threads=2)
    assert origin.tolist() == [float(x) for x in w["out"]]


@pytest.mark.parametrize("dt", DTYPES)
def test_broadcast_autograd_table(oracle, kat, dt):
    """c = a (op) b, backward(error): '+'/'-' reduce the error with the Broadcast implementation (d = index of the
    operand), the other operand replaced by zeros (Addition._autogradBroadcast)."""
    err = np.asarray([5, -2, 7, 3], dtype=dt)
    a = np.asarray([1, 2, 3, 4], dtype=dt)
    for row in kat["broadcast_autograd"]:
        if row["op"] == "*":
            continue  # scalar multiplication: error * b, checked in the GPU autograd test
        bshape = row["b_shape"]
        # rank padding as Permute.makeFit would do for the [2,2] operand: 1-axes go in front
        padded = [1] * (2 - len(bshape)) + list(bshape)
        b = np.resize(np.asarray([8, 9], dtype=dt), int(np.prod(bshape)))
        first, second = (a, b) if row["op"] != "rsub" else (b, a)
        sf, ss = ([2, 2], padded) if row["op"] != "rsub" else (padded, [2, 2])
        op = "-" if row["op"] == "rsub" else row["op"]
        c = np.zeros(4, dtype=dt)
        oracle.broadcast(op, c, ND.of_shape([2, 2]).as_inline_array(), first, ND.of_shape(sf).as_inline_array(), second, ND.of_shape(ss).as_inline_array())
        assert c.tolist() == [float(x) for x in row["c"]], row["src"]
        wrt_b = row["which_grad"] == "b"
        d = (1 if wrt_b else 0) if row["op"] != "rsub" else (0 if wrt_b else 1)
        target_shape = padded if wrt_b else [2, 2]
        other_shape = [2, 2] if wrt_b else padded
        g = np.zeros(int(np.prod(target_shape)), dtype=dt)
        zeros_other = np.zeros(int(np.prod(other_shape)), dtype=dt)
        oracle.broadcast(op, g, ND.of_shape(target_shape).as_inline_array(), zeros_other, ND.of_shape(other_shape).as_inline_array(),
                         err, ND.of_shape([2, 2]).as_inline_array(), d=d)
        assert g.tolist() == [float(x) for x in row["grad"]], row["src"]


def test_sliced_addition(oracle, kat):
    v = kat["sliced_addition"]
    data = np.resize(np.arange(3, 20, dtype=np.float64), 121)
    parent = ND.of_shape([11, 11])
    x = parent.sliced([9, 11], [1, 0], [1, 1])
    y = parent.sliced([9, 11], [0, 0], [1, 1])
    out = np.zeros(99)
    oracle.bielementwise("+", out, ND.of_shape([9, 11]).as_inline_array(), data, x.as_inline_array(), data, y.as_inline_array(), threads=2)
    assert out[:50].tolist() == [float(t) for t in v["first_50"]]


def test_tanh_chain(oracle, kat):
    v = kat["tanh_chain"]
    t = oracle.fun64("tanh", v["x"])
    assert round(t * 100, 4) == v["value_4dp"]
    assert round(oracle.fun64("tanh", v["x"], derive=True) * 100, 4) == v["grad_4dp"]


def test_inline_arrays(kat, oracle):
    for v in kat["inline_arrays"]:
        c = ND.of_shape(v["parent_shape"])
        if v["slice_shape"]:
            c = c.sliced(v["slice_shape"], v["slice_offset"], v["slice_spread"])
        assert c.as_inline_array().tolist() == v["inline"], v["src"]
        for i in range(c.size):
            assert oracle.index_of_index(c.as_inline_array(), i) == c.index_of_index(i)


def test_rng_known_answers(oracle, kat):
    v = kat["fill_randomly"]
    assert oracle.fill_randomly(np.float32, 2, v["seed"]).tolist() == [float(np.float32(x)) for x in v["f32"]]
    # The reference computes the polar multiplier with StrictMath (fdlibm) log/sqrt; glibc's log may round the
    # last bit differently, which moves the F64 values by an ulp or two (the F32 values are unaffected).
    np.testing.assert_allclose(oracle.fill_randomly(np.float64, 2, v["seed"]), v["f64"], rtol=1e-15, atol=0)


def test_gaussian_from_matches_a_java_util_random_stream(oracle):
    """Randomization_Spec.groovy:39-54: gaussianFrom(initialScramble(seed)) equals java.util.Random(seed)'s first
    two nextGaussian() values. The product's generator (nk_jrand_fill) implements java.util.Random itself, so the
    two restatements must agree."""
    import ctypes as C
    from neureka_b200 import _lib as L
    seed = 666_42_666
    scrambled = (seed ^ 0x5DEECE66D) & ((1 << 48) - 1)
    g = oracle.gaussian_from(scrambled)
    out = np.zeros(2)
    assert L.lib.nk_jrand_fill(L.NK_F64, 1, seed, 0.0, 1.0, out.ctypes.data_as(C.c_void_p), 2) == 0
    assert out.tolist() == list(g)


def test_activation_values_at_4(oracle):
    """src/test/groovy/ut/math/Tensor_Function_Spec.groovy:56-90 checks these functions at x = 4 (and -4) to five
    decimals; the values below are the closed forms rounded the same way."""
    import math
    x = 4.0
    expect = {
        "sig": 1 / (1 + math.exp(-x)), "tanh": math.tanh(x), "quad": 16.0, "ln": math.log(x), "relu": 4.0,
        "gaus": math.exp(-16.0), "softplus": math.log(1 + math.exp(x)), "abs": 4.0, "sin": math.sin(x), "cos": math.cos(x),
        "softsign": 0.8, "silu": x / (1 + math.exp(-x)), "exp": math.exp(x), "sqrt": 2.0, "cbrt": 4 ** (1 / 3), "log10": math.log10(4),
    }
    for name, val in expect.items():
        assert oracle.fun64(name, x) == pytest.approx(val, abs=1e-9), name
        assert float(oracle.fun32(name, x)) == pytest.approx(val, rel=1e-6), name
    assert oracle.fun64("relu", -4.0) == pytest.approx(-0.04)


def test_simple_convolution_eligibility(oracle):
    """SimpleCPUConvolution is only taken for dense rank-2/3 operands with a kernel batch of 1."""
    def suit(so, sa, sb, ca=None):
        return oracle.simple_conv_suitable(ND.of_shape(so).as_inline_array(), (ca or ND.of_shape(sa)).as_inline_array(), ND.of_shape(sb).as_inline_array())
    assert suit([252, 252], [256, 256], [5, 5])
    assert suit([4, 6, 6], [4, 8, 8], [1, 3, 3])
    assert not suit([1, 510, 510], [64, 512, 512], [64, 3, 3])       # kernel batch 64
    assert not suit([2, 1, 2], [2, 3, 1], [1, 3, 2])
    assert not suit([2, 2, 2, 2], [3, 3, 3, 3], [2, 2, 2, 2])         # rank 4
    sl = ND.of_shape([9, 9]).sliced([8, 8], [1, 1], [1, 1])
    assert not suit([6, 6], [8, 8], [3, 3], ca=sl)                    # sliced operand -> UNSPECIFIC layout


def test_cpu_sum_tiles(oracle):
    rng = np.random.default_rng(0)
    a = rng.standard_normal(100_000).astype(np.float32)
    s = oracle.cpu_sum(a)
    # 128-wide tiles, recursively, float accumulators
    lvl = a
    while lvl.size > 1:
        n = (lvl.size + 127) // 128
        nxt = np.zeros(n, dtype=np.float32)
        for i in range(n):
            acc = np.float32(0)
            for x in lvl[i * 128:(i + 1) * 128]:
                acc = np.float32(acc + x)
            nxt[i] = acc
        lvl = nxt
    assert np.float32(s) == lvl[0]


def test_matmul_and_dot_restatements_against_the_reference_specs(kat, oracle):
    """CPUMatMul / CPUDot restated (oracle.matmul, oracle.dot) reproduce the values of Matrix_Multiplication_Spec.groovy
    and Tensor_Dot_Product_Spec.groovy exactly, in both item types; on random data they agree with a float64 product
    to the accuracy a rising-order sum in the item type has."""
    for v in kat["matmul"]:
        for dt in (np.float32, np.float64):
            a = np.asarray(v["a"], dtype=dt).reshape(v["M"], v["K"])
            b = np.asarray(v["b"], dtype=dt).reshape(v["K"], v["N"])
            assert oracle.matmul(a, b).reshape(-1).tolist() == v["c"]
    for v in kat["dot"]:
        for dt in (np.float32, np.float64):
            assert oracle.dot(np.asarray(v["a"], dtype=dt), np.asarray(v["b"], dtype=dt)) == v["value"]
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal((33, 70)).astype(np.float32), rng.standard_normal((70, 21)).astype(np.float32)
    want = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(oracle.matmul(a, b) - want).max() <= 70 * 6e-8 * np.abs(want).max() * 4
    # the summation order is the documented one: common index rising, separate multiply and add in the item type
    acc = np.zeros((33, 21), dtype=np.float32)
    for c in range(70):
        acc = acc + (a[:, c:c + 1] * b[c:c + 1, :]).astype(np.float32)
    assert np.array_equal(oracle.matmul(a, b), acc)
    x, y = rng.standard_normal(1003).astype(np.float32), rng.standard_normal(1003).astype(np.float32)
    s = [np.float32(0)] * 4
    for i in range(0, 1000, 4):
        for j in range(4):
            s[j] = np.float32(s[j] + np.float32(x[i + j] * y[i + j]))
    for i in range(1000, 1003):
        s[0] = np.float32(s[0] + np.float32(x[i] * y[i]))
    assert oracle.dot(x, y) == float(np.float32(np.float32(np.float32(s[0] + s[1]) + s[2]) + s[3]))
