"""Halo-split partitioning of a large forward convolution across the GPUs of one box (one process per GPU).

New functionality: the reference has no multi-device execution. A convolution shards along any output dim in
which the image is larger than the kernel (`a_i > b_i`): rank g computes output indices [lo_g, hi_g) of that
dim from the input indices [lo_g, hi_g + b_i - 1) -- its slab plus a halo of b_i - 1 -- so no data is exchanged
while computing. Both the input slab and the output slab are ordinary sliced NDConfigurations of the full
tensors (an offset on the split dim), i.e. exactly the views Neureka's own slicing produces; the assemble step
is therefore "use the owner's output buffer as the drain of nk_conv": results go to their final place over
NVLink with plain stores, or stay local and are gathered with NCCL.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Sequence, Tuple

from .ndconf import NDConfiguration


@dataclass(frozen=True)
class Slab:
    rank: int            # owner
    out_lo: int          # first output index on the split dim
    out_hi: int          # one past the last
    in_lo: int           # first input index (= out_lo)
    in_hi: int           # one past the last input index (= out_hi + halo)

    @property
    def out_len(self) -> int:
        return self.out_hi - self.out_lo

    @property
    def in_len(self) -> int:
        return self.in_hi - self.in_lo


def plan_slabs(out_extent: int, world: int, halo: int) -> List[Slab]:
    """Contiguous, near-equal slabs of the split output dim; earlier ranks take the remainder. Ranks beyond the
    extent get an empty slab."""
    if out_extent < 1 or world < 1 or halo < 0:
        raise ValueError("out_extent and world must be positive, halo non-negative")
    base, rem = divmod(out_extent, world)
    slabs, lo = [], 0
    for g in range(world):
        n = base + (1 if g < rem else 0)
        hi = lo + n
        slabs.append(Slab(g, lo, hi, lo, hi + halo if n > 0 else lo))
        lo = hi
    return slabs


@dataclass(frozen=True)
class GradSlab:
    """A rank's share of the image gradient `D[r] = sum_t k[t] * e[r - t]` along the split dim."""
    rank: int
    lo: int              # first image-gradient index owned
    hi: int              # one past the last
    err_lo: int          # first error index the rank must hold (= lo - halo, clipped)
    err_hi: int          # one past the last error index (= hi, clipped to the error's extent)
    halo: int            # kernel extent - 1

    @property
    def err_len(self) -> int:
        return self.err_hi - self.err_lo

    @property
    def local_extent(self) -> int:
        """Extent of the local deconvolution's drain: error rows held + halo."""
        return self.err_len + (self.halo if self.hi > self.lo else 0)

    @property
    def first_owned_local(self) -> int:
        """Index, inside the local drain, of gradient index `lo` (local index p stands for global err_lo + p)."""
        return self.lo - self.err_lo



def plan_image_grad_slabs(image_extent: int, world: int, halo: int) -> List[GradSlab]:
    """Split of the image gradient of a convolution along a dim where the image (extent a) is larger than the kernel
    (extent b = halo + 1; the error has extent a - halo). Gradient index r needs the error indices r - halo .. r that
    exist, so the halo sits on the error side, *before* the slab. A rank runs the ordinary deconvolution on the error
    rows [err_lo, err_hi) into a local drain of err_len + halo rows; rows [first_owned_local, +hi-lo) of it are
    exact, the other (at most 2 * halo) rows are partial sums that belong to the neighbours and are dropped."""
    if image_extent < 1 or world < 1 or halo < 0 or image_extent - halo < 1:
        raise ValueError("image_extent, world must be positive and the error extent image_extent - halo at least 1")
    err_extent = image_extent - halo
    out = []
    for s in plan_slabs(image_extent, world, 0):
        if s.out_len == 0:
            out.append(GradSlab(s.rank, s.out_lo, s.out_lo, 0, 0, halo))
            continue
        e_lo, e_hi = max(s.out_lo - halo, 0), min(s.out_hi, err_extent)
        if e_hi <= e_lo:   # rows past the error's end that only see its last rows: hold those
            e_lo, e_hi = max(err_extent - 1 - halo, 0), err_extent
        out.append(GradSlab(s.rank, s.out_lo, s.out_hi, e_lo, e_hi, halo))
    return out


def split_dim_for(a_shape: Sequence[int], b_shape: Sequence[int], requested: int = -1) -> int:
    """A dim is splittable when the image is larger than the kernel there (halo b-1; no halo for b == 1). Summed
    dims (a == b) would need a cross-GPU reduction and are refused."""
    if requested >= 0:
        if not a_shape[requested] > b_shape[requested]:
            raise ValueError(f"dim {requested} cannot be halo-split: image extent {a_shape[requested]} is not larger than the kernel's {b_shape[requested]}")
        return requested
    best = max(range(len(a_shape)), key=lambda k: (a_shape[k] > b_shape[k], a_shape[k] - b_shape[k]))
    if not a_shape[best] > b_shape[best]:
        raise ValueError("no dim of this convolution can be halo-split")
    return best


def slab_views(a_shape: Sequence[int], b_shape: Sequence[int], dim: int, slab: Slab) -> Tuple[NDConfiguration, NDConfiguration, Tuple[int, ...]]:
    """(view of the rank's input slab inside the FULL input, view of its output slab inside the FULL output,
    shape of a stand-alone local input slab)."""
    out_shape = [abs(a - b) + 1 for a, b in zip(a_shape, b_shape)]
    in_shape = list(a_shape)
    in_shape[dim] = slab.in_len
    o_shape = list(out_shape)
    o_shape[dim] = slab.out_len
    off_in = [0] * len(a_shape)
    off_in[dim] = slab.in_lo
    off_out = [0] * len(a_shape)
    off_out[dim] = slab.out_lo
    ones = [1] * len(a_shape)
    in_view = NDConfiguration.of_shape(a_shape).sliced(in_shape, off_in, ones)
    out_view = NDConfiguration.of_shape(out_shape).sliced(o_shape, off_out, ones)
    return in_view, out_view, tuple(in_shape)
