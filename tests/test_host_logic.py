"""Host-side logic that needs no GPU: NDConfiguration mirror, expression parser, rank fitting, shapes,
algorithm choice and the backend registration table."""
import numpy as np
import pytest

from neureka_b200.ndconf import Layout, NDConfiguration as ND


def test_layouts_match_the_oracle(oracle):
    rng = np.random.default_rng(1)
    confs = [ND.of_shape(s) for s in ([1], [5], [3, 4], [1, 7], [7, 1], [2, 3, 4], [1, 1, 3], [2, 1, 3, 4])]
    confs += [ND.of_shape(s, Layout.COLUMN_MAJOR) for s in ([3, 4], [2, 3, 4], [1, 5])]
    confs += [ND.of_shape([4, 6]).sliced([3, 4], [1, 0], [1, 1]), ND.of_shape([4, 6]).sliced([2, 2], [0, 1], [2, 2]),
              ND.of_shape([4, 6]).reshaped([1, 0]), ND.of_shape([2, 3, 4]).reshaped([2, 0, 1]), ND.of_shape([3, 4]).reshaped([-1, 0, 1])]
    for c in confs:
        arr = c.as_inline_array()
        assert oracle.layout(arr) == c.layout().value, c
        assert oracle.is_simple(arr) == c.is_simple(), c
        offs = c.element_offsets()
        for i in rng.integers(0, c.size, size=min(c.size, 16)):
            assert oracle.index_of_index(arr, int(i)) == c.index_of_index(int(i)) == offs[i]


def test_specialised_and_general_configurations_agree():
    """NDConfiguration_Spec.groovy:41-127: all configuration classes are the same index function; here there
    is only the general formula, checked against numpy strides."""
    for shape in ([4], [3, 5], [2, 3, 4], [2, 3, 2, 2]):
        c = ND.of_shape(shape)
        ref = np.arange(c.size).reshape(shape)
        assert (c.element_offsets() == ref.reshape(-1)).all()
        perm = list(reversed(range(len(shape))))
        p = c.reshaped(perm)
        assert (p.element_offsets() == ref.transpose(perm).reshape(-1)).all()


def test_construct_validation():
    with pytest.raises(ValueError):
        ND.of([2, 0], [1, 1], [1, 1], [1, 1], [0, 0])
    with pytest.raises(ValueError):
        ND.of([2, 1], [1, 1], [1, 1], [1, 2], [0, 0])


def test_parser_precedence_and_chains():
    from neureka_b200.functions import Function
    assert str(Function.of("i0 x i1")) == "(I[0] x I[1])"
    # 'x' binds looser than '+': the operands of x are the sums
    assert str(Function.of("i0 + i1 x i2")) == "((I[0] + I[1]) x I[2])"
    assert str(Function.of("tanh(i0*i1+i1)")) == "tanh(((I[0] * I[1]) + I[1]))"
    assert str(Function.of("I[0] x>> I[1] x>> I[2]")) == "(I[0] x» I[1] x» I[2])"
    assert str(Function.of("i0<<xi1<<xi2")) == "(I[0] «x I[1] «x I[2])"
    assert str(Function.of("i0 ** i1 / i2")) == "((I[0] ** I[1]) / I[2])"
    with pytest.raises(ValueError):
        Function.of("nope(i0)")


def test_make_fit_and_shapes():
    from neureka_b200.functions import make_fit, shape_of_con, _ends_from
    from neureka_b200.tensor import Tensor
    assert shape_of_con([256, 256], [5, 5]) == (252, 252)
    assert shape_of_con([64, 512, 512], [64, 3, 3]) == (1, 510, 510)
    assert shape_of_con([2, 3, 1], [1, 3, 2]) == (2, 1, 2)
    assert _ends_from([1, 7, 9, 2, 1, 1]) == (1, 2)
    a = Tensor.of(np.float32, [2, 2], [1, 2, 3, 4])
    # [2,2] has no leading/trailing 1-axes -> postfix <= prefix -> padding goes in front
    fit = make_fit([a, Tensor.of(np.float32, [2], [8, 9])])
    assert fit[1].shape == (1, 2)
    # the largest tensor has more trailing than leading 1-axes -> padding goes to the back
    big = Tensor.of(np.float32, [3, 1, 1], [1, 2, 3])
    fit = make_fit([big, Tensor.of(np.float32, [3], [1, 2, 3])])
    assert fit[1].shape == (3, 1, 1)


def test_algorithm_choice():
    from neureka_b200 import backend as B
    from neureka_b200.functions import choose_algorithm
    from neureka_b200.tensor import Tensor
    a = Tensor.of(np.float32, [2, 2], [1, 2, 3, 4])
    assert choose_algorithm(a, Tensor.of(np.float32, [1], [3])) == B.BI_SCALAR_BROADCAST
    assert choose_algorithm(a, Tensor.of(np.float32, [2, 2], 3)) == B.BI_SCALAR_BROADCAST   # virtual
    assert choose_algorithm(a, Tensor.of(np.float32, [2, 2], [1, 1, 1, 1])) == B.BI_ELEMENTWISE
    assert choose_algorithm(a, Tensor.of(np.float32, [2, 1], [1, 1])) == B.BROADCAST


def test_backend_registration_table_mirrors_the_opencl_backend():
    from neureka_b200 import backend as B
    be = B.CudaBackend()
    pairs = set(be.pairs())
    for sym in ["**", "/", "*", "%", "-", "+"]:
        for algo in (B.BI_SCALAR_BROADCAST, B.BROADCAST, B.BI_ELEMENTWISE):
            assert (sym, algo) in pairs
    for sym in ["x", "«x", "x»"]:
        assert (sym, B.ND_CONVOLUTION) in pairs
    assert ("<", B.BI_SCALAR_BROADCAST) in pairs and ("<", B.ELEMENTWISE) in pairs
    from neureka_b200 import _lib as L
    assert len(L.FUN_IDS) == 23
    for f in L.FUN_IDS:
        assert (f, B.ELEMENTWISE) in pairs and (f, B.SCALAR_ALGORITHM) in pairs
    with pytest.raises(L.NeurekaCudaError):
        be.implementation_for("@", "MatMulAlgorithm")


def test_no_cpu_fallback():
    """A call whose operands all live on the host has nowhere to run: the package must refuse, not emulate."""
    from neureka_b200 import _lib as L
    from neureka_b200.functions import Function
    from neureka_b200.tensor import Tensor
    a = Tensor.of(np.float32, [2, 2], [1, 2, 3, 4])
    with pytest.raises(L.NeurekaCudaError):
        Function.of("i0 x i1")(a, a)


def test_reshaping_a_sliced_configuration_resolves_like_a_view_of_its_parent():
    """SimpleReshapeView (config/types/views/SimpleReshapeView.java:96-107) resolves an index by putting the indices
    back into the parent's axis order and asking the parent; its inline array holds the parent's vectors rearranged
    (AbstractNDC.java:182-204). Both descriptions must name the same element for every index -- enumerated here for
    permutations and size-1 paddings of a strided slice."""
    import itertools
    from neureka_b200.ndconf import NDConfiguration as ND

    sl = ND.of_shape([5, 6, 7]).sliced([3, 2, 4], [1, 2, 0], [1, 2, 1])
    for form in ([2, 0, 1], [1, 0, 2], [0, 2, 1], [2, 1, 0], [-1, 2, 0, 1], [1, -1, 0, 2]):
        v = sl.reshaped(form)
        through_parent = []
        for idx in itertools.product(*[range(s) for s in v.shape]):
            inner = [0] * sl.rank
            for i, f in enumerate(form):
                if f >= 0:
                    inner[f] = idx[i]
            through_parent.append(sum((inner[k] * sl.spread[k] + sl.offset[k]) * sl.strides[k] for k in range(sl.rank)))
        assert list(v.element_offsets()) == through_parent, form
        arr = v.as_inline_array()
        r = v.rank
        assert list(arr[:r]) == list(v.shape) and list(arr[r:2 * r]) == list(v.strides)
    import pytest
    with pytest.raises(ValueError):
        sl.reshaped([0, 0, 1])


def test_fused_expression_translation():
    """Function tree -> the expression language of nk_fused_compile: n-ary chains nest to the left like the
    reference's pairwise reduction, unary minus is a multiplication by -1 (FunctionParser), constants are cast to the
    tensor's type, anything that is not elementwise is refused."""
    import pytest
    from neureka_b200.functions import Function, fused_expression_of

    assert fused_expression_of(Function.of("tanh(i0*i1+i1)").root) == ("f_tanh(op_add(op_mul(x0, x1), x1))", 2)
    assert fused_expression_of(Function.of("i0 - i1 - i2").root) == ("op_sub(op_sub(x0, x1), x2)", 3)
    assert fused_expression_of(Function.of("-i0").root) == ("op_mul(T(-1.0), x0)", 1)
    assert fused_expression_of(Function.of("relu(i2) ** 2 % 3").root)[1] == 3          # highest input index + 1
    assert "op_pow(op_pow(" not in fused_expression_of(Function.of("i0 ** 2 / i1").root)[0]
    for bad in ("i0 x i1", "sumItems(i0)", "3 + 4"):
        with pytest.raises(ValueError):
            fused_expression_of(Function.of(bad).root)


def test_bench_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` times the CPU implementation of the same workload and prints one JSON line with the
    keys the driver reads (no GPU needed)."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, os.path.join(root, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                       capture_output=True, text=True, timeout=600, cwd=root)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["metric"] == "nd_conv_gflops" and line["unit"] == "GFLOP/s"
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in line["config"] and "model" not in line["config"]
