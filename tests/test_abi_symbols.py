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


def test_slab_planner_through_the_abi_matches_the_host_planner():
    """nk_group_plan_slabs (what nk_conv_sharded splits with) against neureka_b200.sharding.plan_slabs."""
    from neureka_b200 import _lib as L
    from neureka_b200.sharding import plan_slabs
    for extent, parts, halo in [(2044, 8, 4), (2044, 1, 4), (7, 8, 2), (10, 3, 0), (1, 2, 6), (122, 5, 6)]:
        arrs = [(C.c_int64 * parts)() for _ in range(4)]
        assert L.lib.nk_group_plan_slabs(extent, parts, halo, *arrs) == 0
        want = plan_slabs(extent, parts, halo)
        assert [int(x) for x in arrs[0]] == [s.out_lo for s in want]
        assert [int(x) for x in arrs[1]] == [s.out_len for s in want]
        assert [int(x) for x in arrs[2]] == [s.in_lo for s in want]
        assert [int(x) for x in arrs[3]] == [s.in_len for s in want]
    arrs = [(C.c_int64 * 2)() for _ in range(4)]
    assert L.lib.nk_group_plan_slabs(0, 2, 1, *arrs) == L.NK_ERR_BAD_ARG
    assert L.lib.nk_group_open(None, 0, None) == L.NK_ERR_BAD_ARG


def test_fused_gradient_statements():
    """The statement list handed to nk_fused_compile_grad: one term per occurrence of the input, the error multiplied
    through the tree with one rounding per node."""
    from neureka_b200.functions import Function, fused_gradient_terms_of
    f = Function.of("tanh(i0*i1+i1)", False)
    terms, leaves = fused_gradient_terms_of(f.root, 0)
    assert leaves == 1 and "df_tanh" in terms and terms.rstrip().endswith("term[0] = t4;") and "op_mul(x1, t2)" in terms
    terms, leaves = fused_gradient_terms_of(f.root, 1)
    assert leaves == 2 and "term[0] = t2;" in terms and "op_mul(x0, t2)" in terms
    g = Function.of("i0/i1 - i1**i0", False)
    terms, leaves = fused_gradient_terms_of(g.root, 1)
    assert leaves == 2 and "dop_pow(0, x1, x0)" in terms and "dop_div(1, x0, x1)" in terms and "op_sub(T(0), e)" in terms
    import pytest
    with pytest.raises(ValueError):
        fused_gradient_terms_of(Function.of("relu(i0)", False).root, 1)
