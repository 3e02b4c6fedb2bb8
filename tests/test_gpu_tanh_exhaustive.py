"""Every one of the 2^32 float bit patterns through the device's F32 tanh and sigmoid.

The reference defines tanh on floats as (float)(2 / (1 + Math.exp(-2x)) - 1) evaluated in double
(backend/main/implementations/fun/ScalarTanh.java:24-25). The device evaluates the same sequence of operations with a lean
exp and a Newton reciprocal for |x| >= 2^-26 and literally below (and for NaN); this test is the proof that the float
results are what the reference's formula gives: compared with the CPU oracle's restatement (glibc's exp) on ALL inputs, the
results must agree to one unit in the last place everywhere, NaN exactly where the input is NaN, and differ at all in only
a vanishing share of the inputs (two conforming double exp routines already differ in their last bit now and then, and
that bit decides a float rounding once in millions of inputs).
"""
import numpy as np
import pytest

from neureka_b200 import _lib as L
from neureka_b200.ndconf import NDConfiguration as ND
from helpers import gpu_unary, ulp_diff

pytestmark = pytest.mark.gpu

CHUNK = 1 << 26


def _chunk(i):
    return np.arange(i * CHUNK, (i + 1) * CHUNK, dtype=np.uint64).astype(np.uint32).view(np.float32)


def _sweep(device, oracle, fun, d, step, max_ulp=1):
    """fun (d = -1 forward, 0 derivative) on the bit patterns 0, step, 2 step, ...; returns how many results differ."""
    cfg = ND.of_shape([CHUNK])
    inline = cfg.as_inline_array()
    differing = 0
    want = np.empty(CHUNK, dtype=np.float32)
    for i in range((1 << 32) // (CHUNK * step)):
        x = (np.arange(i * CHUNK, (i + 1) * CHUNK, dtype=np.uint64) * step).astype(np.uint32).view(np.float32)
        got = gpu_unary(device, L.FUN[fun], np.empty(CHUNK, dtype=np.float32), cfg, x, cfg, d=d)
        oracle.unary(fun, want, inline, x, inline, d=d, threads=16)
        gi, wi = got.view(np.int32), want.view(np.int32)
        idx = np.flatnonzero(gi != wi)                      # few, or a block of NaNs whose payloads differ
        if idx.size == 0:
            continue
        nan_w = np.isnan(want[idx])
        assert np.array_equal(np.isnan(got[idx]), nan_w), f"{fun} d={d}: NaN pattern differs in chunk {i}"
        idx = idx[~nan_w]
        if idx.size:
            dd = ulp_diff(got[idx], want[idx])
            assert dd.max() <= max_ulp, f"{fun} d={d} chunk {i}: {dd.max()} ulp at x = {x[idx[int(dd.argmax())]]!r}"
            differing += idx.size
    # the NaN inputs themselves (equal bit patterns pass the filter above only if both sides are NaN or both are not)
    for bits in (0x7fc00000, 0xffc00000, 0x7f800001, 0xff812345):
        x = np.full(16, bits, dtype=np.uint32).view(np.float32)
        c = ND.of_shape([16])
        assert np.isnan(gpu_unary(device, L.FUN[fun], np.zeros(16, dtype=np.float32), c, x, c, d=d)).all()
    return differing


def test_tanh_f32_on_all_float_bit_patterns(device, oracle):
    # measured: a few hundred of 4 294 967 296 differ (by one ulp); the bound leaves room for another libm on the host
    assert _sweep(device, oracle, "tanh", -1, 1) <= 1 << 16


def test_sigmoid_f32_on_all_float_bit_patterns(device, oracle):
    """1 / (1 + Math.exp(-x)) in double (ScalarSigmoid.java), evaluated with the same lean exp and Newton reciprocal."""
    assert _sweep(device, oracle, "sig", -1, 1) <= 1 << 16


@pytest.mark.parametrize("fun", ["silu", "gelu"])
def test_silu_and_gelu_f32_on_every_16th_bit_pattern(device, oracle, fun):
    """x * sig(x) and x * sig(1.702 x) (ScalarSiLU.java, ScalarGeLU.java) on the same sigmoid; -inf gives NaN (-inf * 0)."""
    assert _sweep(device, oracle, fun, -1, 16) <= 1 << 14


def test_tanh_derivative_f32_on_a_dense_sample_of_bit_patterns(device, oracle):
    """tanh' = 1 - tanh(x)^2 with the float-rounded inner tanh (ScalarTanh.java:33-34): every 64th bit pattern."""
    n = 1 << 26
    x = (np.arange(n, dtype=np.uint64) * 64 + 17).astype(np.uint32).view(np.float32)
    cfg = ND.of_shape([n])
    got = gpu_unary(device, L.FUN["tanh"], np.empty(n, dtype=np.float32), cfg, x, cfg, d=0)
    want = np.empty(n, dtype=np.float32)
    oracle.unary("tanh", want, cfg.as_inline_array(), x, cfg.as_inline_array(), d=0, threads=16)
    nan_in = np.isnan(x)
    assert np.array_equal(np.isnan(got), nan_in)
    # 1 - t^2 cancels near |t| = 1: one ulp of the inner tanh moves the result by up to 2^-23 absolute
    ok = np.abs(got[~nan_in].astype(np.float64) - want[~nan_in].astype(np.float64)) <= 2.4e-7
    assert ok.all()
    assert np.count_nonzero(got[~nan_in] != want[~nan_in]) <= n >> 10
