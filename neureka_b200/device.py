"""CudaDevice: the host-side mirror of the `neureka.devices.Device` contract for the CUDA library
(src/main/java/neureka/devices/Device.java:148-216, Storage.java:54-89, AbstractDevice.java:57-208),
i.e. the class that replaces OpenCLDevice's memory handling
(src/main/java/neureka/devices/opencl/OpenCLDevice.java:316-334, 355-405, 497-524, 553-594, 616-632, 676-690).

Device memory is owned by CudaData objects, reference-counted by tensor usage like AbstractDeviceData
(src/main/java/neureka/devices/AbstractDeviceData.java:7-59); slices share their parent's CudaData.
Unlike OpenCLDevice there is no down-cast to F32 on store: F64 is first class.
"""
from __future__ import annotations

import ctypes as C
import weakref
from typing import Dict, Optional

import numpy as np

from . import _lib as L
from .ndconf import NDConfiguration

NP_TO_NK = {
    np.dtype(np.float32): L.NK_F32, np.dtype(np.float64): L.NK_F64, np.dtype(np.int8): L.NK_I8,
    np.dtype(np.int16): L.NK_I16, np.dtype(np.int32): L.NK_I32, np.dtype(np.int64): L.NK_I64,
}


def nk_dtype(dtype) -> int:
    try:
        return NP_TO_NK[np.dtype(dtype)]
    except KeyError:
        raise ValueError(f"data type {dtype} cannot be stored on a CudaDevice") from None


class CudaData:
    """A device allocation; freed when its usage count drops to zero or when it is collected."""

    def __init__(self, device: "CudaDevice", buf: int, size: int, dtype):
        self.device = device
        self.buf = C.c_void_p(buf)
        self.size = int(size)
        self.dtype = np.dtype(dtype)
        self.usages = 0
        self._finalizer = weakref.finalize(self, CudaDevice._release, device, buf)

    def increment_usage(self) -> None:
        self.usages += 1

    def decrement_usage(self) -> None:
        self.usages -= 1
        if self.usages <= 0:
            self.free()

    def free(self) -> None:
        if self._finalizer.alive:
            self._finalizer()

    @property
    def alive(self) -> bool:
        return self._finalizer.alive


class Access:
    """Device.Access (Device.java:305-407): element-offset reads and writes of one tensor's data."""

    def __init__(self, device: "CudaDevice", tensor):
        self._d = device
        self._t = tensor

    def _data(self) -> CudaData:
        d = self._t._data
        if not isinstance(d, CudaData) or d.device is not self._d:
            raise ValueError("tensor is not stored on this device")
        return d

    # write(item).at(i) / .intoRange(start, limit) / .fully()
    def write(self, item):
        data, dev = self._data(), self._d

        class _Writer:
            def into_range(_, start: int, limit: int):
                L.check(L.lib.nk_fill(dev.ctx, data.buf, float(item), start, limit - start), dev.ctx)

            def at(w, index: int):
                w.into_range(index, index + 1)

            def fully(w):
                w.into_range(0, data.size)

        return _Writer()

    # writeFrom(array, offset).intoRange(start, limit) / .fully()
    def write_from(self, array, offset: int = 0):
        data, dev = self._data(), self._d
        arr = np.ascontiguousarray(array, dtype=data.dtype)

        class _Writer:
            def into_range(_, start: int, limit: int):
                if offset < 0 or offset + (limit - start) > arr.size:
                    raise ValueError("source array too small for the requested range")
                L.check(L.lib.nk_write(dev.ctx, data.buf, arr.ctypes.data_as(C.c_void_p), offset, start, limit - start), dev.ctx)

            def at(w, index: int):
                w.into_range(index, index + 1)

            def fully(w):
                w.into_range(0, min(data.size, arr.size - offset))

        return _Writer()

    def read_at(self, index: int):
        return self.read_array(index, 1)[0]

    def read_array(self, start: int, size: int) -> np.ndarray:
        data = self._data()
        out = np.empty(size, dtype=data.dtype)
        L.check(L.lib.nk_read(self._d.ctx, data.buf, out.ctypes.data_as(C.c_void_p), start, size), self._d.ctx)
        return out

    def read_all(self, clone: bool = True) -> np.ndarray:
        return self.read_array(0, self._data().size)

    def get_data_size(self) -> int:
        return self._data().size

    def actualize(self):
        """Virtual (1 element) -> actual (size elements), filled with the single value (OpenCLDevice.java:574-585)."""
        t, dev = self._t, self._d
        old = self._data()
        if old.size >= t.ndconf.size:
            return old
        value = self.read_at(0)
        new = dev.allocate_from_one(old.dtype, t.ndconf.size, value)
        return new

    def virtualize(self):
        """Actual -> virtual: keep only element 0 (OpenCLDevice.java:586-594)."""
        old = self._data()
        value = self.read_at(0)
        return self._d.allocate_from_one(old.dtype, 1, value)


class CudaDevice:
    """One B200 + one stream. `CudaDevice.get(i)` returns the process-wide instance for ordinal i."""

    _instances: Dict[int, "CudaDevice"] = {}

    @staticmethod
    def count() -> int:
        n = C.c_int32(0)
        st = L.lib.nk_device_count(C.byref(n))
        return n.value if st == L.NK_OK else 0

    @classmethod
    def get(cls, ordinal: int = 0) -> "CudaDevice":
        dev = cls._instances.get(ordinal)
        if dev is None or dev.ctx is None:
            dev = cls(ordinal)
            cls._instances[ordinal] = dev
        return dev

    def __init__(self, ordinal: int = 0):
        ctx = C.c_void_p()
        L.check(L.lib.nk_device_open(ordinal, C.byref(ctx)))
        self.ctx: Optional[C.c_void_p] = ctx
        self.ordinal = ordinal
        self._stored = weakref.WeakSet()       # tensors currently on the device
        self._n_data = 0
        props = L.NkProps()
        L.check(L.lib.nk_device_props(self.ctx, C.byref(props)), self.ctx)
        self.props = props
        self.name = props.name.decode()

    # ---- raw allocation ------------------------------------------------------------------------------
    @staticmethod
    def _release(device: "CudaDevice", buf: int) -> None:
        if device.ctx is not None:
            L.lib.nk_free(device.ctx, C.c_void_p(buf))
            device._n_data -= 1

    def _alloc(self, dtype, size: int) -> CudaData:
        buf = C.c_void_p()
        L.check(L.lib.nk_alloc(self.ctx, nk_dtype(dtype), int(size), C.byref(buf)), self.ctx)
        self._n_data += 1
        return CudaData(self, buf.value, size, dtype)

    def allocate(self, dtype, ndc_or_size) -> CudaData:
        """Device.allocate(DataType, NDConfiguration|size) (Device.java:197-201)."""
        size = ndc_or_size.size if isinstance(ndc_or_size, NDConfiguration) else int(ndc_or_size)
        return self._alloc(dtype, size)

    def allocate_from_one(self, dtype, ndc_or_size, initial_value) -> CudaData:
        """Device.allocateFromOne (Device.java:203): every element = initial_value."""
        data = self.allocate(dtype, ndc_or_size)
        L.check(L.lib.nk_fill(self.ctx, data.buf, float(initial_value), 0, data.size), self.ctx)
        return data

    def allocate_from_all(self, dtype, ndc_or_size, array) -> CudaData:
        """Device.allocateFromAll (Device.java:205): upload a whole host array."""
        arr = np.ascontiguousarray(array, dtype=dtype)
        size = ndc_or_size.size if isinstance(ndc_or_size, NDConfiguration) else int(ndc_or_size)
        if arr.size < size:
            raise ValueError("host array smaller than the requested allocation")
        data = self._alloc(dtype, max(size, arr.size))
        L.check(L.lib.nk_write(self.ctx, data.buf, arr.ctypes.data_as(C.c_void_p), 0, 0, arr.size), self.ctx)
        return data

    # ---- Storage contract ----------------------------------------------------------------------------
    def store(self, tensor) -> "CudaDevice":
        """Storage.store (Storage.java:66) -> AbstractDevice.update(ADDED) -> OpenCLDevice._add (:355-405)."""
        if tensor is None:
            raise ValueError("tensor must not be null")
        if self.has(tensor):
            return self
        root = tensor._root()
        if root is not tensor:
            # a slice can only live where its root lives (AbstractDevice.java:92-99): move the root,
            # the slice shares its data
            self.store(root)  # attaches every slice of the root, this one included
            return self
        host = tensor._host_array()
        if tensor.is_virtual:
            data = self.allocate_from_one(tensor.dtype, 1, host[0])
        else:
            data = self.allocate_from_all(tensor.dtype, host.size, host)
        tensor._attach(data, self)
        self._stored.add(tensor)
        for child in tensor._children():
            child._attach(data, self)
            self._stored.add(child)
        if tensor.gradient is not None:  # the gradient migrates with its tensor (OpenCLDevice.java:381-382)
            self.store(tensor.gradient)
        return self

    def restore(self, tensor) -> "CudaDevice":
        """Storage.restore (Storage.java:72) -> OpenCLDevice.restore (:316-334): read all, free, set items."""
        if not self.has(tensor):
            raise ValueError("The given tensor is not stored on this device")
        root = tensor._root()
        host = self.access(root).read_all()
        data = root._data
        root._detach(host)
        for child in root._children():
            child._detach(host)
            self._stored.discard(child)
        self._stored.discard(root)
        data.free()
        if root.gradient is not None and self.has(root.gradient):
            self.restore(root.gradient)
        return self

    def free(self, tensor) -> "CudaDevice":
        """Device.free (Device.java:173): drop the tensor's device data without reading it back."""
        if self.has(tensor):
            data = tensor._data
            tensor._data = None
            tensor.device = None
            self._stored.discard(tensor)
            data.decrement_usage()
        return self

    def has(self, tensor) -> bool:
        return tensor in self._stored and isinstance(tensor._data, CudaData) and tensor._data.device is self

    contains = has

    def number_of_stored(self) -> int:
        return len(self._stored)

    def number_of_data_objects(self) -> int:
        return self._n_data

    def is_empty(self) -> bool:
        return self.number_of_stored() == 0

    def access(self, tensor) -> Access:
        if tensor is None:
            raise ValueError("tensor must not be null")
        return Access(self, tensor)

    def approve(self, call) -> "CudaDevice":
        """Device.approve (Device.java:195): all inputs must live here and share a supported type."""
        for t in call.inputs:
            if t is not None and not self.has(t):
                raise ValueError("every input of a call must be stored on the executing device")
        return self

    def optimized_operation_of(self, function, name):
        """Device.optimizedOperationOf (Device.java:216-241): one run-time compiled kernel for a whole elementwise
        Function (operators + - * / % **, the scalar functions, constants), operands broadcasting against each other.
        Raises ValueError for functions that contain anything else (convolutions, sums)."""
        from .functions import FusedOperation
        return FusedOperation(self, function, name)

    # ---- misc ----------------------------------------------------------------------------------------
    def sync(self) -> None:
        L.check(L.lib.nk_sync(self.ctx), self.ctx)

    def launch_count(self) -> int:
        n = C.c_uint64(0)
        L.check(L.lib.nk_launch_count(self.ctx, C.byref(n)), self.ctx)
        return n.value

    def last_kernel(self) -> str:
        return L.lib.nk_last_kernel(self.ctx).decode()

    def set_conv_path(self, path: int) -> None:
        L.check(L.lib.nk_set_conv_path(self.ctx, path), self.ctx)

    def last_conv_path(self) -> int:
        p = C.c_int32(0)
        L.check(L.lib.nk_last_conv_path(self.ctx, C.byref(p)), self.ctx)
        return p.value

    def dispose(self) -> None:
        """Device.dispose (Device.java:155): restore nothing, release everything."""
        if self.ctx is None:
            return
        for t in list(self._stored):
            self.free(t)
        L.lib.nk_device_close(self.ctx)
        self.ctx = None
        CudaDevice._instances.pop(self.ordinal, None)

    def __repr__(self) -> str:
        return f"CudaDevice[{self.ordinal}: {getattr(self, 'name', '?')}]"
