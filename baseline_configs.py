"""The seeded inputs of the five benchmark configurations, in one place for the tests and the benchmarks.

Rule for a configuration that names one seed for two tensors ("both uniform[-1,1] seed 42"): the tensors are consecutive
pieces of ONE java.util.Random stream of that seed, first operand first. Tensors with seeds of their own start their
own streams. Element order is row-major.
"""
from __future__ import annotations

import numpy as np

from neureka_b200 import jrand

CFG1 = {"a": [256, 256], "k": [5, 5], "out": [252, 252]}
CFG2 = {"a": [64, 512, 512], "k": [64, 3, 3], "out": [1, 510, 510]}
CFG3 = {"a": [4096, 1, 1024], "b": [1, 2048, 1024], "out": [4096, 2048, 1024]}
CFG4 = {"v": [128, 128, 128], "k": [7, 7, 7], "out": [122, 122, 122]}
CFG5 = {"a": [8, 32, 2048, 2048], "k": [1, 32, 5, 5], "out": [8, 1, 2044, 2044]}


def cfg1_inputs():
    """F32 image [256,256] then kernel [5,5], uniform [-1,1], one stream of seed 42."""
    return jrand.stream(np.float32, [256 * 256, 25], jrand.UNIFORM, 42, -1.0, 1.0)


def cfg2_inputs():
    """F32 image [64,512,512] then kernel [64,3,3], N(0,1), one stream of seed 7."""
    return jrand.stream(np.float32, [64 * 512 * 512, 64 * 9], jrand.GAUSSIAN, 7, 0.0, 1.0)


def cfg3_inputs(n: int = 4096, m: int = 2048, k: int = 1024):
    """F32 a [n,1,k] then b [1,m,k], uniform [-2,2], one stream of seed 3 (n, m, k scale the configuration down)."""
    return jrand.stream(np.float32, [n * k, m * k], jrand.UNIFORM, 3, -2.0, 2.0)


def cfg4_inputs():
    """F64 volume [128,128,128] N(0,1) seed 11; kernel [7,7,7] N(0,0.1) seed 12."""
    v = jrand.fill(np.zeros(128 ** 3), jrand.GAUSSIAN, 11, 0.0, 1.0)
    k = jrand.fill(np.zeros(343), jrand.GAUSSIAN, 12, 0.0, 0.1)
    return v, k


def cfg5_kernel():
    """F32 kernel [1,32,5,5], N(0,0.2), seed 6."""
    return jrand.fill(np.zeros(800, dtype=np.float32), jrand.GAUSSIAN, 6, 0.0, 0.2)


def cfg5_image(out: np.ndarray | None = None, start: int = 0, n: int | None = None):
    """F32 image [8,32,2048,2048], uniform [0,1], seed 5: elements start .. start+n of the row-major stream."""
    if out is None:
        out = np.zeros(n if n is not None else 8 * 32 * 2048 * 2048, dtype=np.float32)
    return jrand.fill(out, jrand.UNIFORM, 5, 0.0, 1.0, start)
