"""Slab planner + the multi-rank assemble logic on CPU (gloo, world size 2): every rank convolves its halo slab
(with the CPU oracle standing in for the device) and the gathered slabs must equal the unsharded result."""
import os
import subprocess
import sys

import numpy as np
import pytest

from neureka_b200.sharding import plan_image_grad_slabs, plan_slabs, slab_views, split_dim_for

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


def test_image_gradient_slabs_put_the_halo_on_the_error_side():
    for extent, world, halo in [(2048, 8, 4), (9, 8, 4), (40, 3, 2), (12, 2, 0), (7, 1, 6)]:
        gs = plan_image_grad_slabs(extent, world, halo)
        assert gs[0].lo == 0 and gs[-1].hi == extent
        for g, h in zip(gs, gs[1:]):
            assert g.hi == h.lo
        for g in gs:
            if g.hi == g.lo:
                continue
            assert 0 <= g.err_lo < g.err_hi <= extent - halo
            # every error index a gradient index of the slab needs and that exists is held
            for r in (g.lo, g.hi - 1):
                need = [q for q in range(r - halo, r + 1) if 0 <= q < extent - halo]
                assert all(g.err_lo <= q < g.err_hi for q in need)
            assert g.first_owned_local + (g.hi - g.lo) <= g.local_extent


GRAD_WORKER = r'''
import sys
sys.path.insert(0, sys.argv[1])
import numpy as np
import torch, torch.distributed as dist
from neureka_b200.sharding import plan_image_grad_slabs, plan_slabs
from neureka_b200.ndconf import NDConfiguration as ND
from oracle import oracle as O
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
B, Cn, H, W, KH, KW = 2, 3, 23, 17, 4, 3
OH, OW = H - KH + 1, W - KW + 1
rng = np.random.default_rng(9)
img = rng.standard_normal((B, Cn, H, W)).astype(np.float64)
ker = rng.standard_normal((1, Cn, KH, KW)).astype(np.float64)
err = rng.standard_normal((B, 1, OH, OW)).astype(np.float64)
cf = lambda shape: ND.of_shape(list(shape)).as_inline_array()
# ---- image gradient: rows of the gradient are split, the halo is on the error side --------------------------------------
g = plan_image_grad_slabs(H, world, KH - 1)[rank]
e_loc = np.ascontiguousarray(err[:, :, g.err_lo:g.err_hi, :])
d_loc = np.zeros((B, Cn, g.local_extent, W))
O.conv(d_loc.reshape(-1), cf(d_loc.shape), ker.reshape(-1), cf(ker.shape), e_loc.reshape(-1), cf(e_loc.shape), d=0)
mine = d_loc[:, :, g.first_owned_local:g.first_owned_local + (g.hi - g.lo), :]
# ---- kernel gradient: the forward split; partial sums meet in an all-reduce ------------------------------------------------
f = plan_slabs(OH, world, KH - 1)[rank]
i_loc = np.ascontiguousarray(img[:, :, f.in_lo:f.in_hi, :])
ef_loc = np.ascontiguousarray(err[:, :, f.out_lo:f.out_hi, :])
gk = np.zeros((1, Cn, KH, KW))
O.conv(gk.reshape(-1), cf(gk.shape), i_loc.reshape(-1), cf(i_loc.shape), ef_loc.reshape(-1), cf(ef_loc.shape), d=0)
gk_t = torch.from_numpy(gk)
dist.all_reduce(gk_t)
parts = [None] * world
dist.all_gather_object(parts, mine)
if rank == 0:
    full = np.zeros((B, Cn, H, W))
    O.conv(full.reshape(-1), cf(full.shape), ker.reshape(-1), cf(ker.shape), err.reshape(-1), cf(err.shape), d=0)
    assert np.array_equal(np.concatenate(parts, axis=2), full), "sharded image gradient differs"
    ref_k = np.zeros((1, Cn, KH, KW))
    O.conv(ref_k.reshape(-1), cf(ref_k.shape), img.reshape(-1), cf(img.shape), err.reshape(-1), cf(err.shape), d=0)
    assert np.abs(gk_t.numpy() - ref_k).max() <= 1e-12 * np.abs(ref_k).max()
    print("GRAD_SHARDED_OK")
dist.destroy_process_group()
'''


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_gradients_match_unsharded(tmp_path, world):
    script = tmp_path / "grad_worker.py"
    script.write_text(GRAD_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", str(29720 + world), str(script), ROOT], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "GRAD_SHARDED_OK" in r.stdout


LOCKSTEP_WORKER = r'''
import sys
sys.path.insert(0, sys.argv[1])
import torch, torch.distributed as dist
import bench_sharded as S
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()

# 1. one rank fails while preparing a stage: every rank skips it, nobody enters its collectives
def prepare():
    if rank == 1:
        raise MemoryError("no room on this rank")
    return "ready"
try:
    S._prepared(dist, prepare)
    raise SystemExit("the stage should have been skipped on every rank")
except S.StageSkipped as e:
    assert ("no room" in str(e)) == (rank == 1)

# 2. everybody prepared: a local failure after that point is kept, the rank still enters the stage's collectives
assert S._prepared(dist, lambda: "ready") == "ready"
guard = S._Guard()
calls = []
def launches():
    calls.append(1)
    if rank == 0:
        raise ValueError("refused launch")
for _ in range(3):
    guard.local(launches)                       # raises once on rank 0, is skipped afterwards
    t = torch.ones(4)
    dist.all_reduce(t)                          # every rank is here, every time
    assert float(t[0]) == world
assert len(calls) == (1 if rank == 0 else 3)
assert (guard.error is not None) == (rank == 0)
assert S.agree(dist, guard.error is None) is False   # ... and all ranks report the stage as failed together
assert S.agree(dist, True) is True
print(f"LOCKSTEP_OK {rank}")
dist.destroy_process_group()
'''


def test_a_failing_rank_keeps_its_peers_in_step(tmp_path):
    """bench_sharded's rule for stages with collectives: skip together when a rank fails while preparing, otherwise
    record local failures and keep entering the collectives (gloo, world size 2; no GPU involved)."""
    script = tmp_path / "lockstep_worker.py"
    script.write_text(LOCKSTEP_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
                        "--master-port", "29731", str(script), ROOT], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "LOCKSTEP_OK 0" in r.stdout and "LOCKSTEP_OK 1" in r.stdout
