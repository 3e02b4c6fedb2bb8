"""ctypes binding of libneureka_cuda.so (declared in include/neureka_cuda.h).

The library is the product: there is no CPU fallback. If it is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# NEUREKA_CUDA_LIB points at another build of the same library (e.g. one installed system-wide)
LIB_PATH = os.environ.get("NEUREKA_CUDA_LIB") or os.path.join(_HERE, "lib", "libneureka_cuda.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python -m neureka_b200.build` "
        "(there is no CPU fallback for the CUDA backend)"
    )

lib = C.CDLL(LIB_PATH)

NK_OK, NK_ERR_BAD_ARG, NK_ERR_UNSUPPORTED, NK_ERR_OOM, NK_ERR_CUDA, NK_ERR_TIMEOUT, NK_ERR_BOUNDS = range(7)
NK_F32, NK_F64, NK_I8, NK_I16, NK_I32, NK_I64 = range(6)
NK_OP_ADD, NK_OP_SUB, NK_OP_MUL, NK_OP_DIV, NK_OP_MOD, NK_OP_POW, NK_OP_IDY, NK_OP_MUL_BOTH = range(8)
NK_CONV_AUTO, NK_CONV_GENERIC, NK_CONV_TILED, NK_CONV_TMA, NK_CONV_GEMM, NK_CONV_TC = range(6)
NK_IPC_HANDLE_BYTES = 64

FUN_IDS = [
    "abs", "cbrt", "cos", "exp", "gasu", "gatu", "gaus", "fast_gaus", "gelu", "idy", "log10", "ln",
    "quad", "relu", "selu", "silu", "sig", "sin", "softplus", "softsign", "sqrt", "tanh", "fast_tanh",
]
FUN = {name: i for i, name in enumerate(FUN_IDS)}
OPS = {"+": NK_OP_ADD, "-": NK_OP_SUB, "*": NK_OP_MUL, "/": NK_OP_DIV, "%": NK_OP_MOD, "**": NK_OP_POW}


class NkProps(C.Structure):
    _fields_ = [
        ("name", C.c_char * 256),
        ("total_mem_bytes", C.c_uint64),
        ("sm_count", C.c_int32),
        ("cc_major", C.c_int32),
        ("cc_minor", C.c_int32),
        ("l2_bytes", C.c_int32),
        ("max_smem_per_block", C.c_int32),
        ("clock_khz", C.c_int32),
    ]


_vp, _i32, _i64, _dbl = C.c_void_p, C.c_int32, C.c_int64, C.c_double
_cfg = C.POINTER(C.c_int32)

# name -> (restype, argtypes); every symbol include/neureka_cuda.h declares
SIGNATURES = {
    "nk_device_count": (C.c_int, [C.POINTER(_i32)]),
    "nk_device_open": (C.c_int, [_i32, C.POINTER(_vp)]),
    "nk_device_close": (C.c_int, [_vp]),
    "nk_device_props": (C.c_int, [_vp, C.POINTER(NkProps)]),
    "nk_sync": (C.c_int, [_vp]),
    "nk_stream": (_vp, [_vp]),
    "nk_last_error": (C.c_char_p, [_vp]),
    "nk_version": (C.c_char_p, []),
    "nk_alloc": (C.c_int, [_vp, _i32, _i64, C.POINTER(_vp)]),
    "nk_alloc_shared": (C.c_int, [_vp, _i32, _i64, C.POINTER(_vp)]),
    "nk_wrap": (C.c_int, [_vp, _i32, _vp, _i64, C.POINTER(_vp)]),
    "nk_free": (C.c_int, [_vp, _vp]),
    "nk_buf_info": (C.c_int, [_vp, C.POINTER(_vp), C.POINTER(_i64), C.POINTER(_i32)]),
    "nk_fill": (C.c_int, [_vp, _vp, _dbl, _i64, _i64]),
    "nk_write": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64]),
    "nk_read": (C.c_int, [_vp, _vp, _vp, _i64, _i64]),
    "nk_copy": (C.c_int, [_vp, _vp, _i64, _vp, _i64, _i64]),
    "nk_fused_compile": (C.c_int, [_vp, _i32, _i32, C.c_char_p, C.POINTER(_vp)]),
    "nk_fused_run": (C.c_int, [_vp, _vp, _i32, _vp, _cfg, C.POINTER(_vp), C.POINTER(_cfg)]),
    "nk_fused_free": (C.c_int, [_vp]),
    "nk_fused_compile_grad": (C.c_int, [_vp, _i32, _i32, _i32, _i32, C.c_char_p, C.POINTER(_vp)]),
    "nk_fused_run_grad": (C.c_int, [_vp, _vp, _i32, _vp, _cfg, _vp, _cfg, C.POINTER(_vp), C.POINTER(_cfg)]),
    "nk_probe_wait_timeout": (C.c_int, [_vp, C.c_uint64, C.POINTER(C.c_uint64)]),
    "nk_event_create": (C.c_int, [_vp, C.POINTER(_vp)]),
    "nk_event_record": (C.c_int, [_vp, _vp]),
    "nk_stream_wait_event": (C.c_int, [_vp, _vp]),
    "nk_event_free": (C.c_int, [_vp]),
    "nk_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(_vp)]),
    "nk_host_free": (C.c_int, [_vp]),
    "nk_write_async": (C.c_int, [_vp, _vp, _vp, _i64, _i64, _i64]),
    "nk_read_async": (C.c_int, [_vp, _vp, _vp, _i64, _i64]),
    "nk_conv": (C.c_int, [_vp, _i32, _i32, _vp, _cfg, _vp, _cfg, _vp, _cfg, _i32]),
    "nk_broadcast": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _vp, _cfg, _vp, _cfg, _i32]),
    "nk_binary": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _vp, _cfg, _vp, _cfg, _i32]),
    "nk_unary": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _vp, _cfg, _i32]),
    "nk_scalar_binary": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _vp, _cfg, _dbl, _i32]),
    "nk_fill_fun": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _dbl, _i32]),
    "nk_sum": (C.c_int, [_vp, _i32, _i32, _vp, _cfg, _vp, _i64]),
    "nk_arg_reduce": (C.c_int, [_vp, _i32, _i32, _i32, _vp, _cfg, _vp, _i64]),
    "nk_sum_static": (C.c_int, [_vp, _i32, _i32, _vp, _cfg, _vp, _i64]),
    "nk_set_conv_path": (C.c_int, [_vp, _i32]),
    "nk_last_conv_path": (C.c_int, [_vp, C.POINTER(_i32)]),
    "nk_last_kernel": (C.c_char_p, [_vp]),
    "nk_launch_count": (C.c_int, [_vp, C.POINTER(C.c_uint64)]),
    "nk_timer_begin": (C.c_int, [_vp]),
    "nk_timer_end": (C.c_int, [_vp, C.POINTER(C.c_float)]),
    "nk_measure_fma_peak": (C.c_int, [_vp, _i32, C.POINTER(C.c_double)]),
    "nk_ipc_export": (C.c_int, [_vp, _vp, C.POINTER(C.c_uint8)]),
    "nk_ipc_open": (C.c_int, [_vp, C.POINTER(C.c_uint8), _i32, _i64, C.POINTER(_vp)]),
    "nk_group_open": (C.c_int, [C.POINTER(_i32), _i32, C.POINTER(_vp)]),
    "nk_group_size": (C.c_int, [_vp, C.POINTER(_i32)]),
    "nk_group_ctx": (C.c_int, [_vp, _i32, C.POINTER(_vp)]),
    "nk_group_close": (C.c_int, [_vp]),
    "nk_group_plan_slabs": (C.c_int, [_i64, _i32, _i64, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "nk_conv_sharded": (C.c_int, [_vp, _i32, _i32, C.POINTER(_i64), C.POINTER(_i64), _i32, C.POINTER(_vp), C.POINTER(_vp), _vp]),
    "nk_jrand_fill": (C.c_int, [_i32, _i32, _i64, _dbl, _dbl, _vp, _i64]),
    "nk_jrand_fill_at": (C.c_int, [_i32, _i32, _i64, _dbl, _dbl, _i64, _vp, _i64]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = the library does not export a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class NeurekaCudaError(RuntimeError):
    """Raised for NK_ERR_CUDA / NK_ERR_OOM / NK_ERR_TIMEOUT (the Java glue throws IllegalStateException)."""

    def __init__(self, status: int, message: str):
        super().__init__(f"[nk status {status}] {message}")
        self.status = status


def check(status: int, ctx=None) -> None:
    """Maps a status code to the exception type the reference's implementations throw
    (IllegalArgumentException -> ValueError, IllegalStateException -> NeurekaCudaError)."""
    if status == NK_OK:
        return
    msg = lib.nk_last_error(ctx).decode("utf-8", "replace")
    if status in (NK_ERR_BAD_ARG, NK_ERR_UNSUPPORTED, NK_ERR_BOUNDS):
        raise ValueError(f"[nk status {status}] {msg}")
    if status == NK_ERR_OOM:
        raise MemoryError(f"[nk status {status}] {msg}")
    raise NeurekaCudaError(status, msg)
