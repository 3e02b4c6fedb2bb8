"""A minimal host-side `Tensor` (data + NDConfiguration + device residency + gradient), just enough to
drive the CUDA backend the way Neureka's `Tensor`/`TensorImpl` does
(src/main/java/neureka/Tensor.java, TensorImpl.java:862-865 `to(device)`, :1275-1300 gradients).
Only what the convolution / broadcast / elementwise path needs is mirrored.
"""
from __future__ import annotations

import weakref
from typing import List, Optional, Sequence

import numpy as np

from .ndconf import Layout, NDConfiguration


class Tensor:
    def __init__(self, dtype, ndconf: NDConfiguration, host: Optional[np.ndarray], is_virtual: bool = False):
        self.dtype = np.dtype(dtype)
        self.ndconf = ndconf
        self._host: Optional[np.ndarray] = host   # flat data array while on the host
        self._data = None                          # CudaData while on a device
        self.device = None
        self.is_virtual = is_virtual
        self.is_intermediate = False
        self.rqs_gradient = False
        self.gradient: Optional["Tensor"] = None
        self.graph_node = None
        self._parent: Optional["Tensor"] = None
        self._kids: List[weakref.ref] = []
        self.version = 0

    # ---- factories (Tensor.of(...) overloads) ----------------------------------------------------------
    @staticmethod
    def of(dtype, shape: Sequence[int], data) -> "Tensor":
        """Tensor.of(type, shape, data): a list is repeated cyclically to fill the shape, a scalar gives a
        virtual tensor holding one element (Tensor.java `of(Class, Shape, Object)`)."""
        dtype = np.dtype(dtype)
        shape = tuple(int(s) for s in shape)
        if np.isscalar(data):
            t = Tensor(dtype, NDConfiguration.of_shape(shape), np.full(1, data, dtype=dtype), is_virtual=True)
            return t
        arr = np.asarray(data, dtype=dtype).reshape(-1)
        size = int(np.prod(shape))
        if arr.size != size:
            arr = np.resize(arr, size)
        return Tensor(dtype, NDConfiguration.of_shape(shape), np.ascontiguousarray(arr))

    @staticmethod
    def zeros(dtype, shape) -> "Tensor":
        t = Tensor.of(dtype, shape, 0)
        return t

    @staticmethod
    def like(other: "Tensor", fill=0) -> "Tensor":
        return Tensor.of(other.dtype, other.shape, fill)

    # ---- basic properties ------------------------------------------------------------------------------
    @property
    def shape(self):
        return self.ndconf.shape

    @property
    def rank(self) -> int:
        return self.ndconf.rank

    @property
    def size(self) -> int:
        return self.ndconf.size

    @property
    def is_outsourced(self) -> bool:
        return self.device is not None

    def is_slice(self) -> bool:
        return self._parent is not None

    def set_rqs_gradient(self, flag: bool) -> "Tensor":
        self.rqs_gradient = bool(flag)
        return self

    def set_is_virtual(self, flag: bool) -> "Tensor":
        """MutateTensor.setIsVirtual (TensorImpl.java:290-330): actualize = one element becomes `size` copies."""
        if flag == self.is_virtual:
            return self
        if self._root() is not self:
            raise ValueError("slices cannot change their virtuality")
        if not flag:
            if self.device is not None:
                new = self.device.access(self).actualize()
                old = self._data
                self._swap_data(new)
                old.decrement_usage()
            else:
                self._host = np.full(self.size, self._host[0], dtype=self.dtype)
        else:
            if self.device is not None:
                new = self.device.access(self).virtualize()
                old = self._data
                self._swap_data(new)
                old.decrement_usage()
            else:
                self._host = self._host[:1].copy()
        self.is_virtual = flag
        return self

    # ---- residency -------------------------------------------------------------------------------------
    def _root(self) -> "Tensor":
        t = self
        while t._parent is not None:
            t = t._parent
        return t

    def _children(self) -> List["Tensor"]:
        out = []
        for r in self._kids:
            k = r()
            if k is not None:
                out.append(k)
                out.extend(k._children())
        return out

    def _host_array(self) -> np.ndarray:
        if self._host is None:
            raise ValueError("tensor data is not on the host")
        return self._host

    def _attach(self, data, device) -> None:
        self._data = data
        self.device = device
        self._host = None
        data.increment_usage()

    def _swap_data(self, data) -> None:
        self._data = data
        data.increment_usage()

    def _detach(self, host: np.ndarray) -> None:
        self._data = None
        self.device = None
        self._host = host

    def to(self, device) -> "Tensor":
        """Tensor.to(Device) (TensorImpl.java:862-865); `None` = back to the host (the reference's CPU)."""
        if device is None:
            if self.device is not None:
                self.device.restore(self)
            return self
        if self.device is device:
            return self
        if self.device is not None:
            self.device.restore(self)
        device.store(self)
        return self

    # ---- reading -----------------------------------------------------------------------------------------
    def raw_data(self) -> np.ndarray:
        """The underlying flat data array (mut.data.get())."""
        if self.device is not None:
            return self.device.access(self).read_all()
        return self._host

    @property
    def items(self) -> np.ndarray:
        """All elements in iteration order, resolved through the NDConfiguration (Tensor.getItems)."""
        raw = self.raw_data()
        if self.is_virtual:
            return np.full(self.size, raw[0], dtype=self.dtype)
        return raw[self.ndconf.element_offsets()]

    def item(self, i: int = 0):
        return self.items[i]

    def numpy(self) -> np.ndarray:
        return self.items.reshape(self.shape)

    # ---- views -------------------------------------------------------------------------------------------
    def __getitem__(self, key) -> "Tensor":
        """Slicing: `t[1:3, ::2]` -> Slice._slice (backend/main/operations/other/Slice.java:79-178). The slice
        shares the data of its parent."""
        if not isinstance(key, tuple):
            key = (key,)
        if len(key) != self.rank:
            raise ValueError("one range per axis is required")
        self.set_is_virtual(False)
        new_shape, new_offset, new_spread = [], [], []
        for k, ax in zip(key, self.shape):
            if isinstance(k, int):
                k = slice(k, k + 1, 1)
            start, stop, step = k.indices(ax)
            if step < 1:
                raise ValueError("negative steps are not supported")
            n = len(range(start, stop, step))
            if n < 1:
                raise ValueError("empty slice")
            new_shape.append(n)
            new_offset.append(start)
            new_spread.append(step if n > 1 else 1)
        if self.is_slice():
            raise NotImplementedError("slices of slices are not supported (neither does the reference, Slice.java:156-163)")
        ndc = self.ndconf.sliced(new_shape, new_offset, new_spread)
        sub = Tensor(self.dtype, ndc, self._host)
        sub._parent = self
        self._kids.append(weakref.ref(sub))
        if self.device is not None:
            sub._attach(self._data, self.device)
            self.device._stored.add(sub)
        return sub

    def permute(self, *axes) -> "Tensor":
        """Permute (backend/main/operations/other/Permute.java): a view with rearranged axes; negative
        entries insert axes of size 1."""
        ndc = self.ndconf.reshaped(axes)
        sub = Tensor(self.dtype, ndc, self._host, self.is_virtual)
        sub._parent = self
        self._kids.append(weakref.ref(sub))
        if self.device is not None:
            sub._attach(self._data, self.device)
            self.device._stored.add(sub)
        return sub

    @property
    def T(self) -> "Tensor":
        return self.permute(*reversed(range(self.rank)))

    def to_layout(self, layout: Layout) -> "Tensor":
        """ReLayout.toLayout (backend/main/operations/other/ReLayout.java:66-116): physically rearranges the
        data so that the same logical tensor is stored column- or row-major."""
        cur = self.ndconf.layout()
        if cur is layout or cur is Layout.SYMMETRIC:
            return self
        if layout not in (Layout.ROW_MAJOR, Layout.COLUMN_MAJOR):
            raise ValueError("only ROW_MAJOR and COLUMN_MAJOR are valid targets")
        dev = self.device
        if dev is not None:
            dev.restore(self)
        logical = self.items
        new_conf = NDConfiguration.of_shape(self.shape, layout)
        data = np.zeros(new_conf.required_elements(), dtype=self.dtype)
        data[new_conf.element_offsets()] = logical
        self.ndconf = new_conf
        self._host = data
        if dev is not None:
            dev.store(self)
        return self

    # ---- operators (delegate to the function layer) --------------------------------------------------------
    def _fn(self):
        from . import functions
        return functions

    def conv(self, other):
        return self._fn().Function.of("I[0] x I[1]").call(self, other)

    def __add__(self, o): return self._fn().Function.of("I[0] + I[1]").call(self, self._fn().as_tensor(o, self))
    def __sub__(self, o): return self._fn().Function.of("I[0] - I[1]").call(self, self._fn().as_tensor(o, self))
    def __mul__(self, o): return self._fn().Function.of("I[0] * I[1]").call(self, self._fn().as_tensor(o, self))
    def __truediv__(self, o): return self._fn().Function.of("I[0] / I[1]").call(self, self._fn().as_tensor(o, self))
    def __mod__(self, o): return self._fn().Function.of("I[0] % I[1]").call(self, self._fn().as_tensor(o, self))
    def __pow__(self, o): return self._fn().Function.of("I[0] ** I[1]").call(self, self._fn().as_tensor(o, self))

    def matmul(self, other):
        return self._fn().Function.of("I[0] @ I[1]").call(self, other)

    __matmul__ = matmul

    def sum(self):
        return self._fn().Function.of("sumItems(I[0])").call(self)

    def dot(self, other):
        """Tensor.dot (linear/DotProduct.java): two vectors -> a [1] tensor; differentiable like `x`."""
        from . import autograd
        return autograd.dot(self, other)

    def min(self):
        """Tensor.min (operations/other/Min.java): the smallest item as a [1] tensor; backward puts the error at its index."""
        from . import autograd
        return autograd.extreme(self, False)

    def max(self):
        from . import autograd
        return autograd.extreme(self, True)

    def backward(self, error=None):
        from . import autograd
        autograd.backward(self, error)
        return self

    def __repr__(self) -> str:
        where = "host" if self.device is None else repr(self.device)
        return f"Tensor[{'x'.join(map(str, self.shape))}]({self.dtype}, {where})"
