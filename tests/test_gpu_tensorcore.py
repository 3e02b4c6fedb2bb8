"""The tensor-core (tcgen05, 3xTF32) family for F32 contraction-shaped calls, through nk_conv, against the CPU oracle.

Tolerance: the convolution bound of the path, |gpu - oracle| <= 1e-5 * sum|a||b| per element, no extra factor
(test_gpu_conv.check_conv). The split keeps 22 significant bits per operand, so the error is expected near 1e-6 of
that magnitude; the tests record nothing looser than the stated bound."""
import numpy as np
import pytest

from helpers import gpu_conv
from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND
from test_gpu_conv import check_conv

pytestmark = pytest.mark.gpu
F32 = np.float32


def test_golden_constant_matrix_product_on_the_tensor_cores(device, kat):
    """CrossDeviceSystemTest.java:95-103: [200,300,1] of 2s x [1,300,200] of 3s -> every output 1800, exactly (2 and 3 and
    all partial sums are representable, so the split has nothing to lose)."""
    v = kat["conv_forward_constant"][0]
    a = np.full(int(np.prod(v["a_shape"])), v["a_fill"], dtype=F32)
    b = np.full(int(np.prod(v["b_shape"])), v["b_fill"], dtype=F32)
    co = ND.of_shape(v["out_shape"])
    out = gpu_conv(device, np.zeros(co.size, dtype=F32), co, a, ND.of_shape(v["a_shape"]), b, ND.of_shape(v["b_shape"]), path=L.NK_CONV_TC)
    assert device.last_conv_path() == L.NK_CONV_TC and device.last_kernel().startswith("nk_conv_tc_kernel")
    assert np.all(out == v["out_fill"])


@pytest.mark.parametrize("mkn", [(128, 64, 256), (200, 300, 200), (260, 70, 197), (129, 33, 65), (384, 520, 320), (64, 2000, 64)])
def test_random_contractions_against_the_oracle(device, oracle, mkn):
    m, k, n = mkn
    rng = np.random.default_rng(m * 7 + n)
    a = rng.standard_normal(m * k).astype(F32)
    b = rng.standard_normal(k * n).astype(F32)
    check_conv(device, oracle, F32, ND.of_shape([m, 1, n]), m * n, a, ND.of_shape([m, k, 1]), b, ND.of_shape([1, k, n]), d=-1, path=L.NK_CONV_TC)
    assert device.last_conv_path() == L.NK_CONV_TC


def test_large_products_are_routed_to_the_tensor_cores_by_themselves(device, oracle):
    m, k, n = 512, 256, 512        # 2^26 multiply-adds
    rng = np.random.default_rng(77)
    a = rng.standard_normal(m * k).astype(F32)
    b = rng.standard_normal(k * n).astype(F32)
    c0, c1, c2 = ND.of_shape([m, 1, n]), ND.of_shape([m, k, 1]), ND.of_shape([1, k, n])
    auto = check_conv(device, oracle, F32, c0, m * n, a, c1, b, c2, d=-1)
    assert device.last_conv_path() == L.NK_CONV_TC and device.last_kernel() == "nk_conv_tc_kernel<3xtf32>"
    fma = gpu_conv(device, np.zeros(m * n, dtype=F32), c0, a, c1, b, c2, path=L.NK_CONV_GEMM)
    assert device.last_conv_path() == L.NK_CONV_GEMM
    mag = np.abs(a.reshape(m, k)).astype(np.float64) @ np.abs(b.reshape(k, n)).astype(np.float64)
    assert np.all(np.abs(auto.astype(np.float64) - fma) <= 1e-5 * mag.reshape(-1))
    # F64 has no tensor-core route: the FMA family keeps it
    gpu_conv(device, np.zeros(m * n), c0, a.astype(np.float64), c1, b.astype(np.float64), c2)
    assert device.last_conv_path() == L.NK_CONV_GEMM


def test_roles_swapped_and_several_dims_per_group(device, oracle):
    rng = np.random.default_rng(5)
    for sa, sb in (([1, 64, 300], [180, 64, 1]), ([4, 40, 50, 1, 9], [1, 1, 50, 66, 9]), ([8, 12, 40, 1, 9], [1, 1, 40, 70, 9])):
        so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
        a = rng.standard_normal(int(np.prod(sa))).astype(F32)
        b = rng.standard_normal(int(np.prod(sb))).astype(F32)
        c0 = ND.of_shape(so)
        check_conv(device, oracle, F32, c0, c0.size, a, ND.of_shape(sa), b, ND.of_shape(sb), d=-1, path=L.NK_CONV_TC)


def test_permuted_and_sliced_views(device, oracle):
    """Operands are gathered through offset tables on their way to the K-major panels, the drain is scattered through its
    own: a strided slice, a column-major operand and a drain that is a window of a larger buffer."""
    rng = np.random.default_rng(32)
    M, K, N = 192, 160, 144
    a_full = rng.standard_normal(M * 2 * K).astype(F32)                    # parent [M, 2K, 1]; every second k is used
    b = rng.standard_normal(K * N).astype(F32)
    c1 = ND.of_shape([M, 2 * K, 1]).sliced([M, K, 1], [0, 1, 0], [1, 2, 1])
    c2 = ND.of_shape([N, K, 1]).reshaped([2, 1, 0])                        # B stored as [N, K]: column-major view [1, K, N]
    parent_o = ND.of_shape([M + 3, 1, N + 5])
    c0 = parent_o.sliced([M, 1, N], [2, 0, 4], [1, 1, 1])
    check_conv(device, oracle, F32, c0, parent_o.size, a_full, c1, b, c2, d=-1, path=L.NK_CONV_TC)
    # a transposed drain: [N, 1, M] parent read as [M, 1, N]
    c0t = ND.of_shape([N, 1, M]).reshaped([2, 1, 0])
    check_conv(device, oracle, F32, c0t, M * N, a_full, c1, b, c2, d=-1, path=L.NK_CONV_TC)


@pytest.mark.parametrize("k", [8192, 1000, 136])
def test_long_sums_of_positive_terms_stay_inside_the_bound(device, k):
    """Uniform [0,1) operands and long sums: every term has the same sign, so a biased accumulation shows here first
    (the tensor core truncates when it adds a product block into its accumulator: without the chunked accumulation
    K = 8192 came out 9e-5 low). Reference in float64."""
    m, n = 128, 256
    rng = np.random.default_rng(9)
    a = rng.random(m * k).astype(F32)
    b = rng.random(k * n).astype(F32)
    got = gpu_conv(device, np.zeros(m * n, dtype=F32), ND.of_shape([m, 1, n]), a, ND.of_shape([m, k, 1]), b, ND.of_shape([1, k, n]), path=L.NK_CONV_TC)
    want = a.reshape(m, k).astype(np.float64) @ b.reshape(k, n).astype(np.float64)     # all terms positive: want == sum|a||b|
    rel = np.abs(got.reshape(m, n) - want) / want
    assert rel.max() <= 1e-5, rel.max()


@pytest.mark.parametrize("mkn", [(128, 64, 128), (96, 200, 130)])
def test_both_gradients_of_a_contraction_are_contractions_too(device, oracle, mkn):
    """Convolution.java:56-89: the gradients of y = a x b w.r.t. a and b are deconvolutions of the error with the other
    operand, XConvRight(error, other, zeros) -> nk_conv(drain, other, error, d = 0). For a [M,K,1] x [1,K,N] call both
    are matrix products again (error x b^T and a^T x error) and take the same kernel."""
    m, k, n = mkn
    rng = np.random.default_rng(m + n)
    a = rng.standard_normal(m * k).astype(F32)
    b = rng.standard_normal(k * n).astype(F32)
    e = rng.standard_normal(m * n).astype(F32)
    ca, cb, ce = ND.of_shape([m, k, 1]), ND.of_shape([1, k, n]), ND.of_shape([m, 1, n])
    ga = check_conv(device, oracle, F32, ca, m * k, b, cb, e, ce, d=0, path=L.NK_CONV_TC)     # drain a-shaped, T1 = b, T2 = error
    assert device.last_conv_path() == L.NK_CONV_TC
    gb = check_conv(device, oracle, F32, cb, k * n, a, ca, e, ce, d=0, path=L.NK_CONV_TC)     # drain b-shaped, T1 = a, T2 = error
    assert device.last_conv_path() == L.NK_CONV_TC
    E, A, Bm = e.reshape(m, n).astype(np.float64), a.reshape(m, k).astype(np.float64), b.reshape(k, n).astype(np.float64)
    assert np.abs(ga.reshape(m, k) - E @ Bm.T).max() <= 1e-5 * (np.abs(E) @ np.abs(Bm.T)).max()
    assert np.abs(gb.reshape(k, n) - A.T @ E).max() <= 1e-5 * (np.abs(A.T) @ np.abs(E)).max()
    # AUTO sends these gradient shapes to a contraction family as well once they are worth it (2^21 multiply-adds; the
    # FMA family below 2^24)
    if m * k * n >= (1 << 21):
        gpu_conv(device, np.zeros(m * k, dtype=F32), ca, b, cb, e, ce, d=0)
        assert device.last_conv_path() in (L.NK_CONV_GEMM, L.NK_CONV_TC)


def test_calls_the_family_cannot_take_are_refused_when_forced(device):
    a, b = np.ones(256 * 256, dtype=F32), np.ones(25, dtype=F32)
    with pytest.raises(ValueError):      # a sliding window is not a contraction
        gpu_conv(device, np.zeros(252 * 252, dtype=F32), ND.of_shape([252, 252]), a, ND.of_shape([256, 256]), b, ND.of_shape([5, 5]), path=L.NK_CONV_TC)
    x = np.ones(40 * 16, dtype=F32)
    with pytest.raises(ValueError):      # too small for a 128 x 256 tile to make sense
        gpu_conv(device, np.zeros(40 * 40, dtype=F32), ND.of_shape([40, 1, 40]), x, ND.of_shape([40, 16, 1]), x, ND.of_shape([1, 16, 40]), path=L.NK_CONV_TC)
