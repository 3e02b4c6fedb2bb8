"""Slab planner + the multi-rank assemble logic on CPU (gloo, world size 2): every rank convolves its halo slab
(with the CPU oracle standing in for the device) and the gathered slabs must equal the unsharded result."""
import os
import subprocess
import sys

import numpy as np
import pytest

from neureka_b200.sharding import plan_slabs, slab_views, split_dim_for

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plan_covers_the_output_exactly():
    for extent, world, halo in [(2044, 8, 4), (2044, 1, 4), (7, 8, 2), (10, 3, 0), (1, 2, 6)]:
        slabs = plan_slabs(extent, world, halo)
        assert len(slabs) == world
        assert slabs[0].out_lo == 0 and slabs[-1].out_hi == extent
        for s, t in zip(slabs, slabs[1:]):
            assert s.out_hi == t.out_lo
        assert max(s.out_len for s in slabs) - min(s.out_len for s in slabs) <= 1
        for s in slabs:
            if s.out_len:
                assert s.in_len == s.out_len + halo and s.in_hi <= extent + halo
    with pytest.raises(ValueError):
        plan_slabs(0, 2, 1)


def test_split_dim_choice_and_views():
    a, b = [8, 32, 2048, 2048], [1, 32, 5, 5]
    assert split_dim_for(a, b, 2) == 2
    with pytest.raises(ValueError):
        split_dim_for(a, b, 1)          # the summed channel dim
    assert split_dim_for([64, 512, 512], [64, 3, 3]) in (1, 2)
    slabs = plan_slabs(2044, 8, 4)
    in_view, out_view, local = slab_views(a, b, 2, slabs[3])
    assert in_view.shape == (8, 32, slabs[3].in_len, 2048) and local == in_view.shape
    assert in_view.offset == (0, 0, slabs[3].in_lo, 0)
    assert out_view.shape == (8, 1, slabs[3].out_len, 2044)
    assert out_view.strides == (2044 * 2044, 2044 * 2044, 2044, 1)


WORKER = r'''
import os, sys
sys.path.insert(0, sys.argv[1])
import numpy as np
import torch, torch.distributed as dist
from neureka_b200.sharding import plan_slabs, slab_views
from neureka_b200.ndconf import NDConfiguration as ND
from oracle import oracle as O
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
a_shape, b_shape, dim = [3, 4, 40, 37], [1, 4, 5, 3], 2
rng = np.random.default_rng(5)
a = rng.standard_normal(int(np.prod(a_shape))).astype(np.float32)
b = rng.standard_normal(int(np.prod(b_shape))).astype(np.float32)
out_shape = [abs(x - y) + 1 for x, y in zip(a_shape, b_shape)]
slab = plan_slabs(out_shape[dim], world, b_shape[dim] - 1)[rank]
in_view, out_view, local = slab_views(a_shape, b_shape, dim, slab)
# the rank holds only its slab: gather it out of the full input through the slab view
local_in = np.ascontiguousarray(a[in_view.element_offsets()])
o_shape = list(out_view.shape)
local_out = np.zeros(int(np.prod(o_shape)), dtype=np.float32)
O.conv(local_out, ND.of_shape(o_shape).as_inline_array(), local_in, ND.of_shape(local).as_inline_array(), b, ND.of_shape(b_shape).as_inline_array())
# assemble on rank 0: every rank's slab goes to the place its out_view names
pieces = [None] * world if rank == 0 else None
dist.gather_object((out_view.element_offsets(), local_out), pieces, dst=0)
if rank == 0:
    full = np.zeros(int(np.prod(out_shape)), dtype=np.float32)
    for offs, vals in pieces:
        full[offs] = vals
    ref = np.zeros_like(full)
    O.conv(ref, ND.of_shape(out_shape).as_inline_array(), a, ND.of_shape(a_shape).as_inline_array(), b, ND.of_shape(b_shape).as_inline_array())
    assert np.array_equal(full, ref), "sharded result differs from the unsharded one"
    print("SHARDED_OK")
dist.destroy_process_group()
'''


def test_two_rank_halo_split_matches_unsharded(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29713", str(script), ROOT], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "SHARDED_OK" in r.stdout
