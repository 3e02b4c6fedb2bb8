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
