"""Host-side mirror of Neureka's NDConfiguration (src/main/java/neureka/ndim/config/NDConfiguration.java).

A view of a flat data array = five int vectors of length rank: shape, strides, indicesMap, offset, spread.
    flat i -> nd index : idx_k = i // indicesMap_k ; i %= indicesMap_k           (AbstractNDC / SlicedNDConfiguration.java:93-101)
    nd index -> element: sum_k (idx_k * spread_k + offset_k) * strides_k         (SlicedNDConfiguration.java:103-109)
`as_inline_array()` is the descriptor every kernel entry point of libneureka_cuda takes.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Sequence, Tuple

import numpy as np


class Layout(Enum):
    """NDConfiguration.Layout (NDConfiguration.java:96-146)."""

    ROW_MAJOR = 0
    COLUMN_MAJOR = 1
    SYMMETRIC = 2
    UNSPECIFIC = 3

    def new_strides_for(self, shape: Sequence[int]) -> Tuple[int, ...]:
        """Layout.newStridesFor (NDConfiguration.java:106-129): column major swaps the two leading axes."""
        n = len(shape)
        order = [n - 1 - i for i in range(n)]
        if self is Layout.COLUMN_MAJOR and n > 1:
            order[0], order[1] = order[1], order[0]
        strides = [0] * n
        prod = 1
        for i in order:
            strides[i] = prod
            prod *= shape[i]
        return tuple(strides)

    def rearrange(self, tln: Sequence[int], shape: Sequence[int], new_form: Sequence[int]) -> Tuple[int, ...]:
        """Layout.rearrange (NDConfiguration.java:132-141)."""
        shp_tln = self.new_strides_for(shape)
        return tuple(shp_tln[i] if f < 0 else tln[f] for i, f in enumerate(new_form))


@dataclass(frozen=True)
class NDConfiguration:
    shape: Tuple[int, ...]
    strides: Tuple[int, ...]
    indices_map: Tuple[int, ...]
    spread: Tuple[int, ...]
    offset: Tuple[int, ...]
    virtual: bool = False

    # ---- construction ------------------------------------------------------------------------------
    @staticmethod
    def of(shape, strides, indices_map, spread, offset) -> "NDConfiguration":
        """NDConfiguration.of / AbstractNDC.construct (AbstractNDC.java:68-139): same validation."""
        shape = tuple(int(x) for x in shape)
        if any(d == 0 for d in shape):
            raise ValueError("Shape dimensions must be greater than 0!")
        spread = tuple(int(x) for x in spread)
        for i, d in enumerate(shape):
            if d == 1 and spread[i] > 1:
                raise ValueError(f"A spread/step of {spread[i]} makes no sense for dimension {i} of size 1")
        n = len(shape)
        args = (tuple(int(x) for x in strides), tuple(int(x) for x in indices_map), spread, tuple(int(x) for x in offset))
        if any(len(a) != n for a in args):
            raise ValueError("all five configuration vectors must have the same length")
        return NDConfiguration(shape, *args)

    @staticmethod
    def of_shape(shape, layout: Layout = Layout.ROW_MAJOR) -> "NDConfiguration":
        """The configuration of a freshly created tensor (NDConstructor: row-major strides and indicesMap)."""
        shape = tuple(int(x) for x in shape)
        rm = Layout.ROW_MAJOR.new_strides_for(shape)
        strides = layout.new_strides_for(shape) if layout is Layout.COLUMN_MAJOR else rm
        n = len(shape)
        return NDConfiguration.of(shape, strides, rm, (1,) * n, (0,) * n)

    @staticmethod
    def virtual_of(shape) -> "NDConfiguration":
        """VirtualNDConfiguration (ndim/config/types/views/virtual/VirtualNDConfiguration.java): one element stands for all."""
        shape = tuple(int(x) for x in shape)
        z = (0,) * len(shape)
        return NDConfiguration(shape, z, z, z, z, True)

    # ---- queries -----------------------------------------------------------------------------------
    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def size(self) -> int:
        s = 1
        for d in self.shape:
            s *= d
        return s

    def as_inline_array(self) -> np.ndarray:
        """asInlineArray (NDConfiguration.java:335-345): [shape | strides | indicesMap | offset | spread]."""
        return np.array(self.shape + self.strides + self.indices_map + self.offset + self.spread, dtype=np.int32)

    def is_compact(self) -> bool:
        """isCompact (NDConfiguration.java:386-392)."""
        return all(s in (0, 1) for s in self.spread) and all(o == 0 for o in self.offset)

    def layout(self) -> Layout:
        """getLayout (NDConfiguration.java:157-176)."""
        if not self.is_compact():
            return Layout.UNSPECIFIC
        rm = Layout.ROW_MAJOR.new_strides_for(self.shape)
        cm = Layout.COLUMN_MAJOR.new_strides_for(self.shape)
        has_rm = rm == self.indices_map
        is_rm = rm == self.strides and has_rm
        is_cm = cm == self.strides and has_rm
        if is_rm and is_cm:
            return Layout.SYMMETRIC
        if is_rm:
            return Layout.ROW_MAJOR
        if is_cm:
            return Layout.COLUMN_MAJOR
        return Layout.UNSPECIFIC

    def is_simple(self) -> bool:
        """isSimple (NDConfiguration.java:368-375)."""
        st = self.layout().new_strides_for(self.shape)
        return self.strides == st and self.indices_map == st and self.is_compact()

    def indices_of_index(self, index: int) -> Tuple[int, ...]:
        if self.virtual:
            return (0,) * self.rank
        idx = []
        for m in self.indices_map:
            idx.append(index // m)
            index %= m
        return tuple(idx)

    def index_of_indices(self, indices: Sequence[int]) -> int:
        return sum((indices[i] * self.spread[i] + self.offset[i]) * self.strides[i] for i in range(self.rank))

    def index_of_index(self, index: int) -> int:
        return self.index_of_indices(self.indices_of_index(index))

    def required_elements(self) -> int:
        """Smallest data-array length this view fits into."""
        return 1 + sum(((d - 1) * sp + of) * st for d, sp, of, st in zip(self.shape, self.spread, self.offset, self.strides))

    def element_offsets(self) -> np.ndarray:
        """Data-array position of every element in iteration (row-major) order -- host-side gather map."""
        if self.virtual:
            return np.zeros(self.size, dtype=np.int64)
        off = np.zeros((), dtype=np.int64)
        for k in range(self.rank):
            ax = (np.arange(self.shape[k], dtype=np.int64) * self.spread[k] + self.offset[k]) * self.strides[k]
            off = off[..., None] + ax
        return np.asarray(off).reshape(-1)

    # ---- derived views -----------------------------------------------------------------------------
    def sliced(self, new_shape, new_offset, new_spread) -> "NDConfiguration":
        """Slice._slice (backend/main/operations/other/Slice.java:79-93): parent strides are kept, the
        indicesMap is rebuilt for the new shape, offsets are inherited, a spread of 0 means 1."""
        new_spread = tuple(1 if s == 0 else int(s) for s in new_spread)
        new_offset = tuple(int(o) + self.offset[i] for i, o in enumerate(new_offset))
        lay = self.layout()
        imap = lay.new_strides_for(new_shape)
        return NDConfiguration.of(tuple(new_shape), self.strides, imap, new_spread, new_offset)

    def reshaped(self, new_form: Sequence[int]) -> "NDConfiguration":
        """AbstractNDC._simpleReshape (AbstractNDC.java:182-204): axis permutation / padding with size-1 axes
        (negative entries of new_form). For a configuration that is already sliced or permuted the reference wraps
        the parent in a SimpleReshapeView (config/types/views/SimpleReshapeView.java:60-107), whose five vectors are
        these same rearranged vectors and whose index resolution -- through the parent, with the indices put back in
        the parent's order -- gives exactly sum_i (idx_i * spread_i + offset_i) * strides_i of the rearranged vectors;
        so one construction serves both cases (every parent axis must appear in new_form, as the view demands)."""
        used = sorted(f for f in new_form if f >= 0)
        if used != list(range(self.rank)):
            raise ValueError("a reshape may only permute the axes and pad with size-1 axes: every axis must appear exactly once")
        new_shape = tuple(abs(f) if f < 0 else self.shape[f] for f in new_form)
        lay = self.layout()
        new_strides = lay.rearrange(self.strides, new_shape, new_form)
        new_imap = lay.new_strides_for(new_shape)
        new_spread = tuple(1 if f < 0 else self.spread[f] for f in new_form)
        new_offset = tuple(0 if f < 0 else self.offset[f] for f in new_form)
        return NDConfiguration.of(new_shape, new_strides, new_imap, new_spread, new_offset)
