"""Parity of nk_conv (through the C ABI) with the CPU oracle: golden vectors, random shapes of rank 1..5 over
dense / sliced / strided / column-major / permuted views, F32 and F64, forward and deconvolution.

Tolerances (stated by the task): relative error <= 1e-5 (F32) / <= 1e-12 (F64). "Relative" is taken against the
magnitude the sum can reach, |a|.|b| summed the same way (computed by the oracle on absolute values): that is
the bound that holds for any summation order; a plain max-norm relative check is applied as well."""
import numpy as np
import pytest

from helpers import gpu_conv, rand_view
from neureka_b200 import _lib as L
from neureka_b200.ndconf import Layout, NDConfiguration as ND

pytestmark = pytest.mark.gpu
TOL = {np.dtype(np.float32): 1e-5, np.dtype(np.float64): 1e-12}


def check_conv(device, oracle, dt, c0, n0, a, c1, b, c2, d, path=L.NK_CONV_AUTO):
    dt = np.dtype(dt)
    ref = np.zeros(n0, dtype=dt)
    oracle.conv(ref, c0.as_inline_array(), a, c1.as_inline_array(), b, c2.as_inline_array(), d=d, threads=4)
    scale = np.zeros(n0, dtype=dt)
    oracle.conv(scale, c0.as_inline_array(), np.abs(a), c1.as_inline_array(), np.abs(b), c2.as_inline_array(), d=d, threads=4)
    sentinel = np.full(n0, 777.0, dtype=dt)
    got = gpu_conv(device, sentinel, c0, a, c1, b, c2, d=d, path=path)
    offs = c0.element_offsets()
    untouched = np.ones(n0, dtype=bool)
    untouched[offs] = False
    assert np.all(got[untouched] == 777.0), "elements outside the drain view were written"
    err = np.abs(got[offs].astype(np.float64) - ref[offs].astype(np.float64))
    bound = TOL[dt] * np.maximum(scale[offs].astype(np.float64), np.finfo(dt).tiny)
    assert np.all(err <= bound), f"max err {err.max()} vs bound {bound[err.argmax()]}"
    m = np.abs(ref[offs]).max()
    if m > 0:
        assert err.max() / m <= TOL[dt] * 8
    return got


def check_against_oracle_sampled(oracle, dt, got, c0, a, c1, b, c2, d, rng, n_ranges=6, span=400):
    """The reference's deconvolution scans all of T2 for every drain element, so the oracle is only affordable on
    sampled ranges of a large drain (dense drains only: flat index == data offset)."""
    dt = np.dtype(dt)
    n = c0.size
    span = min(span, n)
    starts = sorted(set([0, n - span] + [int(x) for x in rng.integers(0, n - span + 1, size=n_ranges)]))
    ref, scale = np.zeros(n, dtype=dt), np.zeros(n, dtype=dt)
    for s0 in starts:
        oracle.conv_range(ref, c0.as_inline_array(), a, c1.as_inline_array(), b, c2.as_inline_array(), d, s0, s0 + span)
        oracle.conv_range(scale, c0.as_inline_array(), np.abs(a), c1.as_inline_array(), np.abs(b), c2.as_inline_array(), d, s0, s0 + span)
        seg = slice(s0, s0 + span)
        err = np.abs(got[seg].astype(np.float64) - ref[seg].astype(np.float64))
        bound = TOL[dt] * np.maximum(scale[seg].astype(np.float64), np.finfo(dt).tiny)
        assert np.all(err <= bound), f"max err {err.max()} vs bound {bound[err.argmax()]} in range starting at {s0}"


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_golden_forward(device, kat, dt):
    for v in kat["conv_forward"]:
        out = gpu_conv(device, np.zeros(int(np.prod(v["out_shape"])), dtype=dt), ND.of_shape(v["out_shape"]),
                       np.asarray(v["a"], dtype=dt), ND.of_shape(v["a_shape"]), np.asarray(v["b"], dtype=dt), ND.of_shape(v["b_shape"]))
        assert out.tolist() == [float(x) for x in v["out"]], v["src"]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_golden_constant_matrix_product(device, kat, dt):
    v = kat["conv_forward_constant"][0]
    a = np.full(int(np.prod(v["a_shape"])), v["a_fill"], dtype=dt)
    b = np.full(int(np.prod(v["b_shape"])), v["b_fill"], dtype=dt)
    out = gpu_conv(device, np.zeros(int(np.prod(v["out_shape"])), dtype=dt), ND.of_shape(v["out_shape"]), a, ND.of_shape(v["a_shape"]), b, ND.of_shape(v["b_shape"]))
    assert np.all(out == v["out_fill"])


def test_golden_column_major_and_slice(device, kat):
    v = kat["conv_forward_column_major"][0]
    ca, cb = ND.of_shape(v["a_shape"], Layout.COLUMN_MAJOR), ND.of_shape(v["b_shape"], Layout.COLUMN_MAJOR)
    a_raw, b_raw = np.zeros(6), np.zeros(6)
    a_raw[ca.element_offsets()] = v["a"]
    b_raw[cb.element_offsets()] = v["b"]
    out = gpu_conv(device, np.zeros(9), ND.of_shape(v["out_shape"]), a_raw, ca, b_raw, cb)
    assert out.tolist() == [float(x) for x in v["out"]]
    w = kat["conv_forward_sliced"][0]
    sl = ND.of_shape(w["parent_shape"]).sliced(w["slice_shape"], w["slice_offset"], w["slice_spread"])
    out = gpu_conv(device, np.zeros(1), ND.of_shape([1, 1]), np.asarray(w["parent"], dtype=np.float64), sl, np.asarray(w["b"], dtype=np.float64), ND.of_shape(w["b_shape"]))
    assert out.tolist() == [20.0]


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_golden_xconv_and_autograd_vectors(device, kat, dt):
    v = kat["xconv"][0]
    out = gpu_conv(device, np.zeros(6, dtype=dt), ND.of_shape(v["drain_shape"]), np.asarray(v["t1"], dtype=dt), ND.of_shape(v["t1_shape"]),
                   np.asarray(v["t2"], dtype=dt), ND.of_shape(v["t2_shape"]), d=0)
    assert out.tolist() == [float(x) for x in v["out"]]
    for w in kat["conv_autograd"]:
        g = gpu_conv(device, np.zeros(int(np.prod(w["a_shape"])), dtype=dt), ND.of_shape(w["a_shape"]), np.asarray(w["b"], dtype=dt), ND.of_shape(w["b_shape"]),
                     np.asarray(w["error"], dtype=dt), ND.of_shape(w["error_shape"]), d=0)
        assert g.tolist() == [float(x) for x in w["grad_a"]], w["src"]


def _random_conv_case(rng, rank, max_dim):
    sa, sb = [], []
    for _ in range(rank):
        kind = rng.integers(0, 4)
        big = int(rng.integers(1, max_dim + 1))
        small = int(rng.integers(1, big + 1))
        if kind == 0: sa.append(big); sb.append(big)          # summed dim
        elif kind == 1: sa.append(big); sb.append(small)      # a is the image here
        elif kind == 2: sa.append(small); sb.append(big)      # roles swapped in this dim
        else: sa.append(big); sb.append(1)
    return sa, sb


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("seed", range(6))
def test_random_forward_any_rank_any_view(device, oracle, dt, seed):
    rng = np.random.default_rng(100 + seed)
    kinds = ["dense", "sliced", "strided", "colmajor", "permuted"]
    for trial in range(10):
        rank = int(rng.integers(1, 6))
        sa, sb = _random_conv_case(rng, rank, [40, 12, 8, 6, 5][rank - 1])
        so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
        c1, n1 = rand_view(rng, sa, kinds[int(rng.integers(0, 5))])
        c2, n2 = rand_view(rng, sb, kinds[int(rng.integers(0, 5))])
        c0, n0 = rand_view(rng, so, kinds[int(rng.integers(0, 3))])
        a = rng.standard_normal(n1).astype(dt)
        b = rng.standard_normal(n2).astype(dt)
        check_conv(device, oracle, dt, c0, n0, a, c1, b, c2, d=-1)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("seed", range(4))
def test_random_deconvolution(device, oracle, dt, seed):
    """d >= 0 with arbitrary (even inconsistent) shape triples: whatever the CPU state machine computes, the
    gather kernel must compute too."""
    rng = np.random.default_rng(200 + seed)
    kinds = ["dense", "sliced", "strided", "permuted"]
    for trial in range(10):
        rank = int(rng.integers(1, 5))
        md = [24, 9, 6, 4][rank - 1]
        if trial % 2 == 0:
            # shapes of a real backward pass: forward o = |a-b|+1, then drain := a, t1 := b, t2 := error(o)
            sa, sb = _random_conv_case(rng, rank, md)
            so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
            s0, s1, s2 = (sa, sb, so) if trial % 4 == 0 else (sb, sa, so)
        else:
            s0, s1, s2 = ([int(rng.integers(1, md + 1)) for _ in range(rank)] for _ in range(3))
        c0, n0 = rand_view(rng, s0, kinds[int(rng.integers(0, 3))])
        c1, n1 = rand_view(rng, s1, kinds[int(rng.integers(0, 4))])
        c2, n2 = rand_view(rng, s2, kinds[int(rng.integers(0, 4))])
        t1 = rng.standard_normal(n1).astype(dt)
        t2 = rng.standard_normal(n2).astype(dt)
        check_conv(device, oracle, dt, c0, n0, t1, c1, t2, c2, d=0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_long_reductions_take_the_split_kernel(device, oracle, dt):
    """Few drain elements with long sums (dot products, kernel gradients): the split reduction + finish pass."""
    rng = np.random.default_rng(7)
    n = 250_000   # the reference benchmark's `vector_multiplication`: x of two equal vectors = dot product
    a, b = rng.standard_normal(n).astype(dt), rng.standard_normal(n).astype(dt)
    check_conv(device, oracle, dt, ND.of_shape([1]), 1, a, ND.of_shape([n]), b, ND.of_shape([n]), d=-1)
    assert device.last_kernel() in ("nk_conv_finish_kernel", "nk_conv_reduce_kernel")
    # gradient w.r.t. a small kernel: drain [5,5], t1 = image [64,64], t2 = error [60,60]
    img, err = rng.standard_normal(64 * 64).astype(dt), rng.standard_normal(60 * 60).astype(dt)
    check_conv(device, oracle, dt, ND.of_shape([5, 5]), 25, img, ND.of_shape([64, 64]), err, ND.of_shape([60, 60]), d=0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([96, 200], [5, 5]), ([3, 70, 150], [1, 3, 3]), ([6, 40, 300], [6, 3, 3]), ([2, 5, 64, 130], [1, 5, 5, 5]),
    ([5, 5], [96, 200]), ([20, 33, 140], [3, 7, 7]), ([1, 260], [1, 9]), ([300], [4]), ([40, 256], [40, 3]),
    ([2, 3, 34, 40, 70], [1, 3, 3, 3, 3]),
])
def test_stencil_shapes_all_kernel_families(device, oracle, dt, case):
    """Image-like shapes: AUTO must agree with the oracle and so must every family that accepts the call."""
    rng = np.random.default_rng(11)
    sa, sb = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    b = rng.standard_normal(int(np.prod(sb))).astype(dt)
    c0, c1, c2 = ND.of_shape(so), ND.of_shape(sa), ND.of_shape(sb)
    got = {}
    for path in (L.NK_CONV_AUTO, L.NK_CONV_GENERIC, L.NK_CONV_TILED, L.NK_CONV_TMA):
        try:
            got[path] = check_conv(device, oracle, dt, c0, c0.size, a, c1, b, c2, d=-1, path=path)
        except ValueError as e:
            assert path in (L.NK_CONV_TILED, L.NK_CONV_TMA) and "does not apply" in str(e)
    assert L.NK_CONV_AUTO in got and L.NK_CONV_GENERIC in got


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([3, 6, 333, 700], [1, 6, 5, 5]),      # 108 tiles: no whole wave, every tile cut into units of 16 rows
    ([16, 9, 500, 300], [1, 9, 3, 3]),     # 384 tiles on ~300 CTAs: one whole wave, then the rest in 16-row units
    ([33, 8, 500, 300], [1, 8, 3, 3]),     # F32: 792 tiles, two whole waves, the remaining 200 dealt whole (more than half a tile per CTA)
    ([5, 70, 252], [1, 7, 7]),             # one channel per chunk: the ring-fed kernel
    ([40, 2, 90, 140], [1, 2, 5, 3]),      # many short strips (86 rows each)
])
def test_balanced_walk_gives_the_same_bits_as_one_tile_per_cta(device, oracle, dt, case):
    """The persistent TMA launch (forced here; AUTO walks only from 6 tiles per resident CTA on) runs whole waves of tiles
    and deals the remaining tiles to the CTAs in units of 16 rows, walked in chunks of 2, 4 or 8 rows per warp; the additions
    into one output still come in the same order (channel, window row, window column), so the result must equal the
    one-tile-per-CTA LDGSTS family bit for bit, whatever the tile count -- for the forward call and for the image gradient
    (the same kernel on a padded, flipped problem, weight-loop variant)."""
    rng = np.random.default_rng(41)
    sa, sb = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    b = rng.standard_normal(int(np.prod(sb))).astype(dt)
    c0, c1, c2 = ND.of_shape(so), ND.of_shape(sa), ND.of_shape(sb)
    tma = gpu_conv(device, np.full(c0.size, 777.0, dtype=dt), c0, a, c1, b, c2, path=L.NK_CONV_TMA)
    assert device.last_kernel() in ("nk_conv_tiled_kernel<tma,balanced>", "nk_conv_tiled_kernel<tma,ring>"), device.last_kernel()
    one_tile = gpu_conv(device, np.full(c0.size, -1.0, dtype=dt), c0, a, c1, b, c2, path=L.NK_CONV_TILED)
    assert device.last_kernel() == "nk_conv_tiled_kernel<ldgsts>"
    assert np.array_equal(tma, one_tile)
    rngs = np.random.default_rng(42)
    check_against_oracle_sampled(oracle, dt, tma, c0, a, c1, b, c2, -1, rngs, n_ranges=4, span=300)
    # image gradient: drain image-shaped, T1 = kernel, T2 = error
    e = rng.standard_normal(c0.size).astype(dt)
    grad = gpu_conv(device, np.full(c1.size, 777.0, dtype=dt), c1, b, c2, e, c0, d=0)
    if (so[-1] * np.dtype(dt).itemsize) % 16 == 0:
        assert device.last_conv_path() == L.NK_CONV_TMA
    generic = gpu_conv(device, np.zeros(c1.size, dtype=dt), c1, b, c2, e, c0, d=0, path=L.NK_CONV_GENERIC)
    check_against_oracle_sampled(oracle, dt, grad, c1, b, c2, e, c0, 0, rngs, n_ranges=3, span=40)
    assert np.abs(grad - generic).max() <= (1e-5 if dt == np.float32 else 1e-12) * np.abs(generic).max() * 4


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_gradients_of_tensors_whose_rows_no_tensor_map_can_describe(device, oracle, dt):
    """Rows of 127 and 125 elements are no multiple of 16 bytes in either type, so neither the image nor the error can be
    given to a tensor map as it lies. Both gradients must still run on the TMA families -- on a copy with rows padded to
    16 bytes -- and agree with the gather family and (sampled) with the oracle."""
    rng = np.random.default_rng(77)
    sa, sb = [8, 8, 70, 127], [1, 8, 3, 3]
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    b = rng.standard_normal(int(np.prod(sb))).astype(dt)
    e = rng.standard_normal(int(np.prod(so))).astype(dt)
    c0, c1, c2 = ND.of_shape(so), ND.of_shape(sa), ND.of_shape(sb)
    tol = 1e-5 if dt == np.float32 else 1e-12
    rngs = np.random.default_rng(78)
    # image gradient: drain image-shaped, T1 = kernel, T2 = error
    grad = gpu_conv(device, np.full(c1.size, 777.0, dtype=dt), c1, b, c2, e, c0, d=0)
    assert device.last_conv_path() == L.NK_CONV_TMA and device.last_kernel().startswith("nk_conv_tiled_kernel<tma"), device.last_kernel()
    generic = gpu_conv(device, np.zeros(c1.size, dtype=dt), c1, b, c2, e, c0, d=0, path=L.NK_CONV_GENERIC)
    assert np.abs(grad - generic).max() <= tol * np.abs(generic).max() * 4
    check_against_oracle_sampled(oracle, dt, grad, c1, b, c2, e, c0, 0, rngs, n_ranges=3, span=40)
    # kernel gradient: drain kernel-shaped, T1 = image, T2 = error
    gk = gpu_conv(device, np.full(c2.size, 777.0, dtype=dt), c2, a, c1, e, c0, d=0)
    assert device.last_conv_path() == L.NK_CONV_TMA and device.last_kernel() == "nk_conv_wgrad_finish_kernel", device.last_kernel()
    gk_generic = gpu_conv(device, np.zeros(c2.size, dtype=dt), c2, a, c1, e, c0, d=0, path=L.NK_CONV_GENERIC)
    assert np.abs(gk - gk_generic).max() <= tol * 8 * np.abs(gk_generic).max()
    # the same tensors as strided views of wider parents: still one padded copy, same numbers
    par = np.zeros([8, 1, 68, 200], dtype=dt)
    par[..., 3:128] = e.reshape(so)
    cpar = ND.of_shape([8, 1, 68, 200]).sliced(so, [0, 0, 0, 3], [1, 1, 1, 1])
    grad_v = gpu_conv(device, np.full(c1.size, 777.0, dtype=dt), c1, b, c2, par.ravel(), cpar, d=0)
    assert np.array_equal(grad_v, grad)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([32, 64, 256], [32, 3, 3], 8), ([16, 70, 132], [16, 5, 5], 4), ([24, 50, 260], [24, 3, 3], 6),
    ([2, 16, 40, 128], [1, 16, 3, 3], 4), ([64, 40, 256], [64, 3, 3], 16),
])
def test_channel_split_adds_up_inside_a_cluster(device, oracle, dt, case):
    """Few tiles, many channels: the channel range is split over CTAs. Up to 8 parts form one thread-block cluster
    that adds its partial tiles through distributed shared memory (one launch); more parts take the two-pass path.
    Both must agree with the oracle, and with each other bit for bit (same summation order)."""
    rng = np.random.default_rng(23)
    sa, sb, parts = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    b = rng.standard_normal(int(np.prod(sb))).astype(dt)
    c0, c1, c2 = ND.of_shape(so), ND.of_shape(sa), ND.of_shape(sb)
    for path in (L.NK_CONV_TMA, L.NK_CONV_TILED):
        check_conv(device, oracle, dt, c0, c0.size, a, c1, b, c2, d=-1, path=path)
        kernel = device.last_kernel()
        if parts <= 8:
            assert kernel.endswith("cluster>"), kernel
        else:
            assert kernel == "nk_conv_tiled_finish_kernel", kernel


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([96, 200], [5, 5]), ([3, 70, 150], [1, 3, 3]), ([6, 40, 300], [6, 3, 3]), ([2, 5, 64, 130], [1, 5, 5, 5]),
    ([20, 33, 140], [3, 7, 7]), ([1, 260], [1, 9]), ([40, 256], [40, 3]), ([2, 3, 34, 40, 70], [1, 3, 3, 3, 3]), ([16, 24, 72], [7, 7, 7]),
])
def test_image_gradient_as_padded_correlation(device, oracle, dt, case):
    """Gradient of a convolution w.r.t. its image: XConvRight(error, kernel, zeros(image shape)) -> the implementation
    sees (drain = image-shaped, T1 = kernel, T2 = error) with d = 0. AUTO routes it to the zero-padded, flipped
    TMA correlation; it must agree with the oracle's deconvolution and with the generic gather family."""
    rng = np.random.default_rng(13)
    sa, sb = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    k = rng.standard_normal(int(np.prod(sb))).astype(dt)
    e = rng.standard_normal(int(np.prod(so))).astype(dt)
    c0, c1, c2 = ND.of_shape(sa), ND.of_shape(sb), ND.of_shape(so)
    auto = gpu_conv(device, np.zeros(c0.size, dtype=dt), c0, k, c1, e, c2, d=0)
    family = device.last_conv_path()
    generic = gpu_conv(device, np.zeros(c0.size, dtype=dt), c0, k, c1, e, c2, d=0, path=L.NK_CONV_GENERIC)
    assert device.last_conv_path() == L.NK_CONV_GENERIC
    check_against_oracle_sampled(oracle, dt, auto, c0, k, c1, e, c2, 0, rng)
    # a tensor map needs the error's row stride to be a multiple of 16 bytes; other shapes stay on the gather family
    row_bytes = so[-1] * np.dtype(dt).itemsize
    if row_bytes % 16 == 0:
        assert family == L.NK_CONV_TMA, "the image gradient did not take the tiled path"
    scale = np.abs(generic).max()
    assert np.abs(auto - generic).max() <= (1e-5 if dt == np.float32 else 1e-12) * scale * 4


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([300, 520], [5, 5]), ([3, 70, 150], [1, 3, 3]), ([4, 8, 100, 260], [1, 8, 5, 5]), ([64, 64, 64], [7, 7, 7]),
    ([2, 1040], [1, 5]), ([6, 130, 264], [6, 3, 3]), ([40, 72, 136], [3, 7, 7]),
])
def test_kernel_gradient_reduction(device, oracle, dt, case):
    """Gradient of a convolution w.r.t. its kernel: (drain = kernel-shaped, T1 = image, T2 = error), d = 0: few
    outputs, each a sum over the whole error. AUTO may take the TMA reduction kernel; it must agree with the oracle's
    deconvolution and with the generic family."""
    rng = np.random.default_rng(17)
    sa, sb = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    e = rng.standard_normal(int(np.prod(so))).astype(dt)
    c0, c1, c2 = ND.of_shape(sb), ND.of_shape(sa), ND.of_shape(so)
    auto = check_conv(device, oracle, dt, c0, c0.size, a, c1, e, c2, d=0)
    family, kernel = device.last_conv_path(), device.last_kernel()
    generic = gpu_conv(device, np.zeros(c0.size, dtype=dt), c0, a, c1, e, c2, d=0, path=L.NK_CONV_GENERIC)
    isz = np.dtype(dt).itemsize
    eligible = (so[-1] * isz) % 16 == 0 and (sa[-1] * isz) % 16 == 0 and int(np.prod(so)) >= 65536 and so[-1] >= 64
    if eligible:
        assert family == L.NK_CONV_TMA and kernel == "nk_conv_wgrad_finish_kernel", (family, kernel)
    scale = np.abs(generic).max()
    assert np.abs(auto - generic).max() <= (1e-5 if dt == np.float32 else 1e-12) * scale * 16


@pytest.mark.parametrize("dt", [np.float32, np.float64])
@pytest.mark.parametrize("case", [
    ([200, 300, 1], [1, 300, 200]),            # CrossDeviceSystemTest.java:95-103, Tensor.convDot
    ([260, 70, 1], [1, 70, 197]),              # ragged tile edges
    ([1, 64, 300], [180, 64, 1]),              # roles swapped: the output rows come from the second operand
    ([4, 40, 50, 1, 9], [1, 1, 50, 33, 9]),    # several dims per index group: M = 160, N = 33, K = 450
    ([64, 40, 1], [1, 40, 64]),                # under 2^21 multiply-adds: not worth the tables -> gather family
    ([257, 33], [1, 33]),                      # N = 1: not a matrix product worth tiling -> stays on the gather family
])
def test_contractions_take_the_gemm_family(device, oracle, dt, case):
    """Calls in which every dim is summed away or spanned by one operand only are dense contractions
    O[m,n] = sum_k A[m,k] B[k,n]; AUTO routes the large ones to the register-tiled GEMM kernel, which must agree with the
    oracle's state machine and with the gather family."""
    rng = np.random.default_rng(31)
    sa, sb = case
    so = [abs(x - y) + 1 for x, y in zip(sa, sb)]
    a = rng.standard_normal(int(np.prod(sa))).astype(dt)
    b = rng.standard_normal(int(np.prod(sb))).astype(dt)
    c0, c1, c2 = ND.of_shape(so), ND.of_shape(sa), ND.of_shape(sb)
    auto = check_conv(device, oracle, dt, c0, c0.size, a, c1, b, c2, d=-1)
    family = device.last_conv_path()
    m = int(np.prod([x for x, y in zip(sa, sb) if y == 1 and x > 1] or [1]))
    n = int(np.prod([y for x, y in zip(sa, sb) if x == 1 and y > 1] or [1]))
    k = int(np.prod([x for x, y in zip(sa, sb) if x == y] or [1]))
    big = min(m, n) >= 32 and k >= 16 and m * n * k >= (1 << 21)
    assert (family == L.NK_CONV_GEMM) == bool(big), family
    if big:
        assert device.last_kernel() == "nk_conv_gemm_kernel"
    generic = gpu_conv(device, np.zeros(c0.size, dtype=dt), c0, a, c1, b, c2, d=-1, path=L.NK_CONV_GENERIC)
    tol = 1e-5 if dt == np.float32 else 1e-12
    assert np.abs(auto - generic).max() <= tol * np.abs(generic).max() * 8


def test_gemm_family_on_permuted_and_sliced_views(device, oracle):
    """The contraction kernel gathers through offset tables, so column-major operands, a strided slice and a drain
    that is a window of a larger buffer must give the same numbers as the dense case."""
    rng = np.random.default_rng(32)
    M, K, N = 192, 160, 144
    a_full = rng.standard_normal(M * 2 * K).astype(np.float32)             # parent [M, 2K, 1]; every second k is used
    b = rng.standard_normal(K * N).astype(np.float32)
    c1 = ND.of_shape([M, 2 * K, 1]).sliced([M, K, 1], [0, 1, 0], [1, 2, 1])
    c2 = ND.of_shape([N, K, 1]).reshaped([2, 1, 0])                        # B stored as [N, K]: column-major view [1, K, N]
    parent_o = ND.of_shape([M + 3, 1, N + 5])
    c0 = parent_o.sliced([M, 1, N], [2, 0, 4], [1, 1, 1])
    got = check_conv(device, oracle, np.float32, c0, parent_o.size, a_full, c1, b, c2, d=-1)
    assert device.last_conv_path() == L.NK_CONV_GEMM
    a2 = a_full.reshape(M, 2 * K)[:, 1::2].astype(np.float64)
    b2 = b.reshape(N, K).T.astype(np.float64)
    want = a2 @ b2
    view = got.reshape(M + 3, N + 5)[2:2 + M, 4:4 + N]
    assert np.abs(view - want).max() <= 1e-5 * np.abs(a2).max() * np.abs(b2).max() * K


def test_tiled_family_on_views(device, oracle):
    """Sliced image with an offset (unaligned rows), a drain that is a slice of a larger output (the multi-GPU
    assemble writes that way) and a column-major kernel."""
    rng = np.random.default_rng(5)
    for dt in (np.float32, np.float64):
        parent = ND.of_shape([4, 70, 203])
        c1 = parent.sliced([4, 64, 199], [0, 3, 1], [1, 1, 1])
        c2 = ND.of_shape([4, 3, 5])
        out_parent = ND.of_shape([1, 80, 200])
        c0 = out_parent.sliced([1, 62, 195], [0, 9, 2], [1, 1, 1])
        a = rng.standard_normal(parent.size).astype(dt)
        b = rng.standard_normal(c2.size).astype(dt)
        check_conv(device, oracle, dt, c0, out_parent.size, a, c1, b, c2, d=-1)


def test_argument_errors_are_reported_not_faulted(device):
    dt = np.float32
    a, b = np.ones(16, dtype=dt), np.ones(4, dtype=dt)
    with pytest.raises(ValueError, match="reaches elements"):
        gpu_conv(device, np.zeros(4, dtype=dt), ND.of_shape([3, 3]), a, ND.of_shape([4, 4]), b, ND.of_shape([2, 2]))
    with pytest.raises(ValueError, match="drain extent"):
        gpu_conv(device, np.zeros(16, dtype=dt), ND.of_shape([4, 4]), a, ND.of_shape([4, 4]), b, ND.of_shape([2, 2]))
    with pytest.raises(ValueError, match="rank"):
        gpu_conv(device, np.zeros(1, dtype=dt), ND.of_shape([1] * 9), np.ones(1, dtype=dt), ND.of_shape([1] * 9), np.ones(1, dtype=dt), ND.of_shape([1] * 9))
