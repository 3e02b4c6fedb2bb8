"""ctypes wrapper of the CPU oracle (oracle/oracle.cpp). TEST INFRASTRUCTURE ONLY: it may be imported by
tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs, never by the product package.
Tensors are passed as (numpy data array, inline configuration array)."""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

F32, F64 = 0, 1
OP = {"+": 0, "-": 1, "*": 2, "/": 3, "%": 4, "**": 5, "idy": 6, "test_mul": 7}
FUN_IDS = [
    "abs", "cbrt", "cos", "exp", "gasu", "gatu", "gaus", "fast_gaus", "gelu", "idy", "log10", "ln",
    "quad", "relu", "selu", "silu", "sig", "sin", "softplus", "softsign", "sqrt", "tanh", "fast_tanh",
]
FUN = {n: i for i, n in enumerate(FUN_IDS)}


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "oracle.cpp")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _SO


def _load():
    build()
    lib = C.CDLL(_SO)
    vp, i32, i64, dbl = C.c_void_p, C.c_int32, C.c_int64, C.c_double
    cfg = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
    lib.orc_conv.argtypes = [i32, i32, vp, cfg, vp, cfg, vp, cfg, i32, i32, i32]
    lib.orc_conv_range.argtypes = [i32, i32, vp, cfg, vp, cfg, vp, cfg, i32, i64, i64]
    lib.orc_simple_conv_suitable.argtypes = [i32, cfg, cfg, cfg]
    lib.orc_broadcast.argtypes = [i32, i32, vp, cfg, vp, cfg, vp, cfg, i32, i32, i32]
    lib.orc_bielementwise.argtypes = [i32, i32, vp, cfg, vp, cfg, vp, cfg, i32, i32, i32]
    lib.orc_scalar_broadcast.argtypes = [i32, i32, vp, cfg, vp, cfg, dbl, i32, i32, i32]
    lib.orc_unary.argtypes = [i32, i32, vp, cfg, vp, cfg, i32, i32, i32]
    lib.orc_fun64.argtypes = [i32, i32, dbl]
    lib.orc_fun64.restype = dbl
    lib.orc_fun32.argtypes = [i32, i32, C.c_float]
    lib.orc_fun32.restype = C.c_float
    lib.orc_sum.argtypes = [i32, vp, i64]
    lib.orc_sum.restype = dbl
    lib.orc_matmul.argtypes = [i32, vp, vp, vp, i64, i64, i64]
    lib.orc_dot.argtypes = [i32, vp, vp, i64]
    lib.orc_dot.restype = dbl
    lib.orc_layout.argtypes = [i32, cfg]
    lib.orc_is_simple.argtypes = [i32, cfg]
    lib.orc_index_of_index.argtypes = [i32, cfg, i64]
    lib.orc_index_of_index.restype = i64
    lib.orc_gaussian_from.argtypes = [i64, C.POINTER(dbl)]
    lib.orc_fill_randomly.argtypes = [i32, vp, i64, i64]
    return lib


_lib = _load()


def _dt(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return F32
    if a.dtype == np.float64:
        return F64
    raise TypeError(f"oracle supports float32/float64, got {a.dtype}")


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def _cfg(c) -> np.ndarray:
    return np.ascontiguousarray(c, dtype=np.int32)


def conv(drn, cfg0, s1, cfg1, s2, cfg2, d=-1, threads=1, allow_simple=True) -> int:
    """AbstractCPUConvolution.run: returns 1 when the SimpleCPUConvolution fast path was taken."""
    rank = len(cfg0) // 5
    r = _lib.orc_conv(_dt(drn), rank, _p(drn), _cfg(cfg0), _p(s1), _cfg(cfg1), _p(s2), _cfg(cfg2), d, threads, int(allow_simple))
    if r < 0:
        raise ValueError("oracle conv failed")
    return r


def conv_range(drn, cfg0, s1, cfg1, s2, cfg2, d, start, end) -> None:
    rank = len(cfg0) // 5
    r = _lib.orc_conv_range(_dt(drn), rank, _p(drn), _cfg(cfg0), _p(s1), _cfg(cfg1), _p(s2), _cfg(cfg2), d, start, end)
    if r < 0:
        raise ValueError("oracle conv_range failed")


def simple_conv_suitable(cfg0, cfg1, cfg2) -> bool:
    return bool(_lib.orc_simple_conv_suitable(len(cfg0) // 5, _cfg(cfg0), _cfg(cfg1), _cfg(cfg2)))


def broadcast(op, drn, cfg0, a, cfg1, b, cfg2, d=-1, threads=1) -> None:
    _lib.orc_broadcast(_dt(drn), len(cfg0) // 5, _p(drn), _cfg(cfg0), _p(a), _cfg(cfg1), _p(b), _cfg(cfg2), OP[op], d, threads)


def bielementwise(op, drn, cfg0, a, cfg1, b, cfg2, d=-1, threads=1) -> None:
    _lib.orc_bielementwise(_dt(drn), len(cfg0) // 5, _p(drn), _cfg(cfg0), _p(a), _cfg(cfg1), _p(b), _cfg(cfg2), OP[op], d, threads)


def scalar_broadcast(op, drn, cfg0, a, cfg1, value, d=-1, threads=1) -> None:
    _lib.orc_scalar_broadcast(_dt(drn), len(cfg0) // 5, _p(drn), _cfg(cfg0), _p(a), _cfg(cfg1), float(value), OP[op], d, threads)


def unary(fun, drn, cfg0, a, cfg1, d=-1, threads=1) -> None:
    r = _lib.orc_unary(_dt(drn), len(cfg0) // 5, _p(drn), _cfg(cfg0), _p(a), _cfg(cfg1), FUN[fun], d, threads)
    if r < 0:
        raise ValueError("oracle unary failed")


def fun64(fun, x, derive=False) -> float:
    return _lib.orc_fun64(FUN[fun], int(derive), float(x))


def fun32(fun, x, derive=False) -> np.float32:
    return np.float32(_lib.orc_fun32(FUN[fun], int(derive), float(np.float32(x))))


def cpu_sum(a: np.ndarray) -> float:
    a = np.ascontiguousarray(a)
    return _lib.orc_sum(_dt(a), _p(a), a.size)


def matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """CPUMatMul on dense row-major matrices [M,K] @ [K,N] (F32 or F64), the reference's summation order."""
    assert a.dtype == b.dtype and a.ndim == 2 and b.ndim == 2 and a.shape[1] == b.shape[0]
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    out = np.zeros((a.shape[0], b.shape[1]), dtype=a.dtype)
    _lib.orc_matmul(_dt(a), _p(out), _p(a), _p(b), a.shape[0], a.shape[1], b.shape[1])
    return out


def dot(a: np.ndarray, b: np.ndarray) -> float:
    """CPUDot on two vectors of one type (DOT.unrolled04's four partial sums)."""
    assert a.dtype == b.dtype and a.size == b.size
    a, b = np.ascontiguousarray(a).reshape(-1), np.ascontiguousarray(b).reshape(-1)
    return float(_lib.orc_dot(_dt(a), _p(a), _p(b), a.size))


def layout(cfg) -> int:
    return _lib.orc_layout(len(cfg) // 5, _cfg(cfg))


def is_simple(cfg) -> bool:
    return bool(_lib.orc_is_simple(len(cfg) // 5, _cfg(cfg)))


def index_of_index(cfg, i) -> int:
    return _lib.orc_index_of_index(len(cfg) // 5, _cfg(cfg), i)


def gaussian_from(seed: int):
    out = (C.c_double * 2)()
    _lib.orc_gaussian_from(seed, out)
    return out[0], out[1]


def fill_randomly(dtype, n: int, seed: int) -> np.ndarray:
    a = np.zeros(n, dtype=dtype)
    _lib.orc_fill_randomly(_dt(a), _p(a), n, seed)
    return a
