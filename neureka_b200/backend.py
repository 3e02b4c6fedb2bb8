"""CudaBackend: the registration table that puts a CUDA `ImplementationFor` on every
(Operation, Algorithm) pair of the path, mirroring CLBackend._load
(src/main/java/neureka/backend/ocl/CLBackend.java:200-325), and the implementations themselves -- thin
adapters from an ExecutionCall to one C-ABI kernel call, like CLConvolution / CLBroadcast /
CLBiElementwise / CLElementwiseFunction / CLScalarBroadcast are for OpenCL.

Conventions of ImplementationFor.run (src/main/java/neureka/backend/api/ImplementationFor.java:56-72):
input(0) is the pre-allocated drain, already on the device; input(1..) are the sources; the derivative
index < 0 means forward; the implementation returns input(0) and signals failure by raising.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np

from . import _lib as L
from .device import CudaDevice, nk_dtype
from .tensor import Tensor

# algorithm names (src/main/java/neureka/backend/main/algorithms/*.java)
ND_CONVOLUTION = "NDConvolution"
BROADCAST = "Broadcast"
BI_ELEMENTWISE = "BiElementwise"
BI_SCALAR_BROADCAST = "BiScalarBroadcast"
ELEMENTWISE = "ElementwiseAlgorithm"
SCALAR_ALGORITHM = "ScalarAlgorithm"
SCALAR_BROADCAST = "ScalarBroadcast"
SUM_ALGORITHM = "SumAlgorithm"
MIN_ALGORITHM, MAX_ALGORITHM = "min_algorithm", "max_algorithm"
DOT_ALGORITHM = "DotProductAlgorithm"

OPERATORS = ["**", "/", "*", "%", "-", "+"]                       # Power ... Addition
CONV_OPS = ["x", "«x", "x»"]                            # Convolution, XConvLeft, XConvRight
ASSIGN_LEFT = "<"


@dataclass
class ExecutionCall:
    """ExecutionCall (src/main/java/neureka/backend/api/ExecutionCall.java): inputs + DerivIdx + operation + device."""

    inputs: List[Optional[Tensor]]
    operation: str
    device: CudaDevice
    deriv_idx: int = -1
    args: Dict[str, object] = field(default_factory=dict)

    def input(self, i: int) -> Optional[Tensor]:
        return self.inputs[i]

    @property
    def arity(self) -> int:
        return len(self.inputs)

    def with_input_at(self, i: int, t: Optional[Tensor]) -> "ExecutionCall":
        ins = list(self.inputs)
        ins[i] = t
        return ExecutionCall(ins, self.operation, self.device, self.deriv_idx, dict(self.args))

    def with_added_input_at(self, i: int, t: Optional[Tensor]) -> "ExecutionCall":
        ins = list(self.inputs)
        ins.insert(i, t)
        return ExecutionCall(ins, self.operation, self.device, self.deriv_idx, dict(self.args))

    def rearrange_inputs(self, *order: int) -> None:
        self.inputs = [self.inputs[i] for i in order]


def _cfg(t: Tensor):
    arr = t.ndconf.as_inline_array()
    return arr, arr.ctypes.data_as(C.POINTER(C.c_int32))


def _same_type(call: ExecutionCall, n: int) -> int:
    dt = call.input(0).dtype
    for i in range(1, n):
        if call.input(i).dtype != dt:
            raise ValueError("all tensors of a call must have the same item type")
    return nk_dtype(dt)


class ImplementationFor:
    def run(self, call: ExecutionCall) -> Tensor:  # pragma: no cover - interface
        raise NotImplementedError


class CudaConvolution(ImplementationFor):
    """Replaces CLConvolution (implementations/convolution/CLConvolution.java:10-32)."""

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        t0, t1, t2 = call.input(0), call.input(1), call.input(2)
        for t in (t1, t2):
            t.set_is_virtual(False)  # AbstractCPUConvolution.java:42-43
        dt = _same_type(call, 3)
        k0, c0 = _cfg(t0); k1, c1 = _cfg(t1); k2, c2 = _cfg(t2)
        L.check(L.lib.nk_conv(dev.ctx, dt, t0.rank, t0._data.buf, c0, t1._data.buf, c1, t2._data.buf, c2, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaBroadcast(ImplementationFor):
    """Replaces CLBroadcast* (implementations/broadcast/CLBroadcast.java:10-33)."""

    def __init__(self, op: int):
        self.op = op

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        t0, t1, t2 = call.input(0), call.input(1), call.input(2)
        t0.set_is_virtual(False)  # CPUBroadcast.java:37
        for t in (t1, t2):
            t.set_is_virtual(False)
        dt = _same_type(call, 3)
        k0, c0 = _cfg(t0); k1, c1 = _cfg(t1); k2, c2 = _cfg(t2)
        L.check(L.lib.nk_broadcast(dev.ctx, self.op, dt, t0.rank, t0._data.buf, c0, t1._data.buf, c1, t2._data.buf, c2, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaBiElementwise(ImplementationFor):
    """Replaces CLBiElementwise* (implementations/elementwise/CLBiElementwise.java:7-32)."""

    def __init__(self, op: int):
        self.op = op

    def run(self, call: ExecutionCall) -> Tensor:
        if call.arity < 3:
            raise ValueError("The element-wise operation requires at least two arguments and one output!")
        dev = call.device
        t0, t1, t2 = call.input(0), call.input(1), call.input(2)
        for t in (t1, t2):
            t.set_is_virtual(False)  # CPUBiElementWise.java:59-60
        dt = _same_type(call, 3)
        k0, c0 = _cfg(t0); k1, c1 = _cfg(t1); k2, c2 = _cfg(t2)
        L.check(L.lib.nk_binary(dev.ctx, self.op, dt, t0.rank, t0._data.buf, c0, t1._data.buf, c1, t2._data.buf, c2, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaScalarBroadcast(ImplementationFor):
    """Replaces CLScalarBroadcast* (implementations/broadcast/CLScalarBroadcast.java:16-64): drain = f(src, value),
    the value being element 0 of the last input."""

    def __init__(self, op: int):
        self.op = op

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        offset = 1 if call.arity == 3 else 0
        t0, src, scalar = call.input(0), call.input(offset), call.input(1 + offset)
        value = float(dev.access(scalar).read_at(0)) if dev.has(scalar) else float(scalar._host_array()[0])
        src.set_is_virtual(False)
        t0.set_is_virtual(False)
        dt = nk_dtype(t0.dtype)
        k0, c0 = _cfg(t0); k1, c1 = _cfg(src)
        L.check(L.lib.nk_scalar_binary(dev.ctx, self.op, dt, t0.rank, t0._data.buf, c0, src._data.buf, c1, value, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaElementwiseFunction(ImplementationFor):
    """Replaces CLElementwiseFunction (implementations/elementwise/CLElementwiseFunction.java:12-42)."""

    def __init__(self, fun: int):
        self.fun = fun

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        t0, t1 = call.input(0), call.input(1)
        t1.set_is_virtual(False)  # CLElementwiseFunction.java:32
        dt = _same_type(call, 2)
        k0, c0 = _cfg(t0); k1, c1 = _cfg(t1)
        L.check(L.lib.nk_unary(dev.ctx, self.fun, dt, t0.rank, t0._data.buf, c0, t1._data.buf, c1, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaScalarFunction(ImplementationFor):
    """ScalarAlgorithm (algorithms/ScalarAlgorithm.java:17-53; CLScalarFunction.java:19-27): a one-element
    tensor in, a one-element tensor out. Evaluated by the device's own scalar code, not on the host."""

    def __init__(self, fun: int):
        self.fun = fun

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        t0, t1 = call.input(0), call.input(1)
        value = float(dev.access(t1).read_at(0))
        k0, c0 = _cfg(t0)
        L.check(L.lib.nk_fill_fun(dev.ctx, self.fun, nk_dtype(t0.dtype), t0.rank, t0._data.buf, c0, value, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaScalarBroadcastFunction(ImplementationFor):
    """ScalarBroadcast (algorithms/ScalarBroadcast.java:65-82): every element of the drain := fun(scalar)."""

    def __init__(self, fun: int):
        self.fun = fun

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        t0, t1 = call.input(0), call.input(1)
        value = float(dev.access(t1).read_at(0)) if dev.has(t1) else float(t1._host_array()[0])
        t0.set_is_virtual(False)
        k0, c0 = _cfg(t0)
        L.check(L.lib.nk_fill_fun(dev.ctx, self.fun, nk_dtype(t0.dtype), t0.rank, t0._data.buf, c0, value, call.deriv_idx), dev.ctx)
        t0.version += 1
        return t0


class CudaSum(ImplementationFor):
    """Replaces CLSum (operations/linear/internal/opencl/CLSum.java:23-132): input(0) or input(1) -> a new [1] tensor."""

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        src = call.input(0) if call.input(0) is not None else call.input(1)
        src.set_is_virtual(False)
        out = Tensor.of(src.dtype, (1,), [0])
        dev.store(out)
        k, c = _cfg(src)
        L.check(L.lib.nk_sum(dev.ctx, nk_dtype(src.dtype), src.rank, src._data.buf, c, out._data.buf, 0), dev.ctx)
        return out


class CudaReduce(ImplementationFor):
    """Replaces CLReduce (operations/linear/internal/opencl/CLReduce.java:34-147; CPU twin operations/other/internal/CPUReduce.java):
    the flat index of the smallest / largest element as a [1] tensor of ints."""

    def __init__(self, want_max: bool):
        self.want_max = 1 if want_max else 0

    def run(self, call: ExecutionCall) -> Tensor:
        dev = call.device
        src = call.input(0) if call.input(0) is not None else call.input(1)
        src.set_is_virtual(False)
        out = Tensor.of(np.int32, (1,), [0])
        dev.store(out)
        k, c = _cfg(src)
        L.check(L.lib.nk_arg_reduce(dev.ctx, self.want_max, nk_dtype(src.dtype), src.rank, src._data.buf, c, out._data.buf, 0), dev.ctx)
        return out


class CudaBackend:
    """BackendExtension for the CUDA device (src/main/java/neureka/backend/api/BackendExtension.java:15-70).

    `implementation_for(operation, algorithm)` is DeviceAlgorithm.getImplementationFor(CudaDevice.class)."""

    def __init__(self):
        self._table: Dict[Tuple[str, str], ImplementationFor] = {}
        self._load()

    def _set(self, operation: str, algorithm: str, impl: ImplementationFor) -> None:
        self._table[(operation, algorithm)] = impl

    def _load(self) -> None:
        # same pair list as CLBackend._load (CLBackend.java:200-325), minus MatMul/DotProduct/Randomization
        for sym in OPERATORS:
            op = L.OPS[sym]
            self._set(sym, BI_SCALAR_BROADCAST, CudaScalarBroadcast(op))
            self._set(sym, BROADCAST, CudaBroadcast(op))
            self._set(sym, BI_ELEMENTWISE, CudaBiElementwise(op))
        self._set(ASSIGN_LEFT, BI_SCALAR_BROADCAST, CudaScalarBroadcast(L.NK_OP_IDY))
        self._set(ASSIGN_LEFT, ELEMENTWISE, CudaElementwiseFunction(L.FUN["idy"]))
        for sym in CONV_OPS:
            self._set(sym, ND_CONVOLUTION, CudaConvolution())
        for name, fid in L.FUN.items():
            self._set(name, ELEMENTWISE, CudaElementwiseFunction(fid))
            self._set(name, SCALAR_ALGORITHM, CudaScalarFunction(fid))
            self._set(name, SCALAR_BROADCAST, CudaScalarBroadcastFunction(fid))
        self._set("sumItems", SUM_ALGORITHM, CudaSum())
        self._set("min", MIN_ALGORITHM, CudaReduce(False))
        self._set("max", MAX_ALGORITHM, CudaReduce(True))
        # DotProduct (linear/DotProduct.java; CLDot / CPUDot): two vectors of one length are the `x` call whose single dim
        # is summed away -- the convolution implementation serves it (its long-reduction kernel)
        self._set("dot", DOT_ALGORITHM, CudaConvolution())

    def implementation_for(self, operation: str, algorithm: str) -> ImplementationFor:
        try:
            return self._table[(operation, algorithm)]
        except KeyError:
            # OpenCLDevice.getKernel throws IllegalStateException for a missing kernel (OpenCLDevice.java:709-713)
            raise L.NeurekaCudaError(L.NK_ERR_UNSUPPORTED, f"no CUDA implementation registered for operation '{operation}' / algorithm '{algorithm}'") from None

    def pairs(self):
        return sorted(self._table.keys())

    @staticmethod
    def find(key: str) -> Optional[CudaDevice]:
        """BackendExtension.find (BackendExtension.java:40-48): 'cuda', 'gpu', 'nvidia', 'first', an ordinal, or
        'cuda:<ordinal>' / 'gpu:<ordinal>' for one of several GPUs in this process."""
        key = key.strip().lower()
        n = CudaDevice.count()
        if n == 0:
            return None
        if key.startswith(("cuda:", "gpu:")):
            key = key.split(":", 1)[1]
        if key.isdigit():
            return CudaDevice.get(int(key)) if int(key) < n else None
        if key in ("cuda", "gpu", "nvidia", "first", "any", "b200"):
            return CudaDevice.get(0)
        return None


_BACKEND: Optional[CudaBackend] = None


def backend() -> CudaBackend:
    global _BACKEND
    if _BACKEND is None:
        _BACKEND = CudaBackend()
    return _BACKEND
