"""The C-ABI library loads without a GPU and exports every symbol include/neureka_cuda.h declares."""
import ctypes as C
import os
import re

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "neureka_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(nk_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    from neureka_b200 import _lib as L
    names = _declared()
    assert len(names) >= 35
    for n in names:
        assert hasattr(L.lib, n), f"{n} is declared in the header but not exported"
        assert n in L.SIGNATURES, f"{n} has no ctypes signature"
    assert sorted(L.SIGNATURES) == names


def test_version_and_error_reporting_without_a_device():
    from neureka_b200 import _lib as L
    assert b"sm_100a" in L.lib.nk_version()
    # invalid handles are rejected with a message, not a crash
    assert L.lib.nk_sync(None) == L.NK_ERR_BAD_ARG
    assert b"invalid context" in L.lib.nk_last_error(None)
    assert L.lib.nk_free(None, None) == L.NK_OK


def test_jrand_streams():
    """java.util.Random semantics: nextFloat = 24 bits, nextDouble = 26+27 bits; first values of seed 42 are the
    well-known 0.7275637 / 0.7275636800328681."""
    from neureka_b200 import _lib as L
    f = np.zeros(3, dtype=np.float32)
    d = np.zeros(2, dtype=np.float64)
    assert L.lib.nk_jrand_fill(L.NK_F32, 0, 42, 0.0, 1.0, f.ctypes.data_as(C.c_void_p), 3) == 0
    assert L.lib.nk_jrand_fill(L.NK_F64, 0, 42, 0.0, 1.0, d.ctypes.data_as(C.c_void_p), 2) == 0
    assert f[0] == np.float32(0.7275637)
    assert d[0] == 0.7275636800328681
    assert 0 <= f.min() and f.max() < 1
    g = np.zeros(100_000, dtype=np.float64)
    assert L.lib.nk_jrand_fill(L.NK_F64, 1, 7, 0.0, 1.0, g.ctypes.data_as(C.c_void_p), g.size) == 0
    assert abs(g.mean()) < 0.02 and abs(g.std() - 1) < 0.02
    assert L.lib.nk_jrand_fill(9, 0, 1, 0.0, 1.0, g.ctypes.data_as(C.c_void_p), 1) == L.NK_ERR_UNSUPPORTED


def test_host_only_generator_library_matches_the_cuda_library_and_splits_one_stream():
    """libnk_jrand.so (no CUDA inside) draws the same streams as the generator exported by the CUDA library, and
    two tensors that share a seed are consecutive pieces of one stream."""
    from neureka_b200 import _lib as L
    from neureka_b200 import jrand
    import baseline_configs as B
    for dt, code in ((np.float32, L.NK_F32), (np.float64, L.NK_F64)):
        for dist, p0, p1 in ((0, -2.0, 2.0), (1, 0.0, 0.2)):
            want = np.zeros(1000, dtype=dt)
            assert L.lib.nk_jrand_fill(code, dist, 7, p0, p1, want.ctypes.data_as(C.c_void_p), want.size) == 0
            assert np.array_equal(jrand.fill(np.zeros(1000, dtype=dt), dist, 7, p0, p1), want)
    a, b = B.cfg3_inputs(8, 4, 16)
    one = jrand.fill(np.zeros(8 * 16 + 4 * 16, dtype=np.float32), jrand.UNIFORM, 3, -2.0, 2.0)
    assert np.array_equal(np.concatenate([a, b]), one)
    # a jump into the uniform stream lands on the same elements
    assert np.array_equal(jrand.fill(np.zeros(50, dtype=np.float32), jrand.UNIFORM, 3, -2.0, 2.0, start=128), one[128:178])
    a1, k1 = B.cfg1_inputs()
    assert a1.size == 65536 and k1.size == 25 and np.abs(a1).max() <= 1.0


def test_fused_plan_switches_to_64_bit_counters_before_32_bit_ones_can_wrap():
    from neureka_b200 import _lib as L
    wide = L.lib.nk_fused_plan_is_wide
    grid = 148 * 16
    assert wide(1000, 2000, grid) == 0
    assert wide((1 << 32) - grid - 1, 1000, grid) == 0
    assert wide((1 << 32) - grid, 1000, grid) == 1          # the unit counter steps by the grid size past 2^32
    assert wide(1 << 31, (1 << 32) - 2, grid) == 1            # the second row of the last group: row index 2^32 - 1 + 1
    assert wide(1 << 31, (1 << 32) - 3, grid) == 0
    assert wide(1 << 33, 1 << 34, grid) == 1
