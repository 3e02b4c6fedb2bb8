"""java.util.Random-compatible input streams (csrc/nk_jrand.cpp) from a host-only library.

libnk_jrand.so holds nothing but the generator, so a process that must stay off the GPU (the CPU arm of the benchmark)
can draw the seeded inputs without mapping the CUDA library. The same two functions are also exported by
libneureka_cuda.so (include/neureka_cuda.h: nk_jrand_fill, nk_jrand_fill_at).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "lib", "libnk_jrand.so")
if not os.path.exists(_PATH):
    from .build import build_jrand
    build_jrand()
_lib = C.CDLL(_PATH)
_lib.nk_jrand_fill.restype = C.c_int
_lib.nk_jrand_fill.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_double, C.c_double, C.c_void_p, C.c_int64]
_lib.nk_jrand_fill_at.restype = C.c_int
_lib.nk_jrand_fill_at.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_double, C.c_double, C.c_int64, C.c_void_p, C.c_int64]

UNIFORM, GAUSSIAN = 0, 1
_DT = {np.dtype(np.float32): 0, np.dtype(np.float64): 1}


def fill(out: np.ndarray, dist: int, seed: int, p0: float, p1: float, start: int = 0) -> np.ndarray:
    """Fills the contiguous float array `out` with elements start .. start+out.size of the stream of `seed`:
    uniform on [p0, p1) (dist 0) or Gaussian with mean p0 and deviation p1 (dist 1, start must be 0)."""
    assert out.flags["C_CONTIGUOUS"]
    st = _lib.nk_jrand_fill_at(_DT[out.dtype], dist, seed, p0, p1, start, out.ctypes.data_as(C.c_void_p), out.size)
    if st != 0:
        raise ValueError(f"nk_jrand_fill_at: status {st}")
    return out


def fill_ptr(ptr, dtype, n: int, dist: int, seed: int, p0: float, p1: float, start: int = 0) -> None:
    st = _lib.nk_jrand_fill_at(_DT[np.dtype(dtype)], dist, seed, p0, p1, start, ptr, n)
    if st != 0:
        raise ValueError(f"nk_jrand_fill_at: status {st}")


def stream(dtype, sizes, dist: int, seed: int, p0: float, p1: float):
    """Tensors that share a seed are consecutive pieces of ONE stream, in the order given."""
    total = int(sum(sizes))
    both = fill(np.zeros(total, dtype=dtype), dist, seed, p0, p1)
    out, pos = [], 0
    for n in sizes:
        out.append(both[pos:pos + n].copy())
        pos += n
    return out
