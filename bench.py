#!/usr/bin/env python
"""Benchmark of the convolution hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl cuda|reference] [--assemble copy|peer|nccl] [--scale S]

Workload (config.workload): BASELINE config 5 -- the 4-D F32 convolution a[8,32,2048,2048] (uniform [0,1], seed 5)
x k[1,32,5,5] (N(0,0.2), seed 6) -> [8,1,2044,2044], 53.48 GFLOP and 4.43 GB of algorithmic traffic per pass; it is the
largest single-GPU configuration and the one that shards. With N > 1 (one process per GPU, launched by torchrun)
the output rows (dim 2) are halo-split over the ranks; each rank holds its input slab (+4 halo rows). The result is
assembled in rank 0's memory in one of three ways: `copy` (default) -- every rank computes into a local slab and a
second stream pushes the finished slab into rank 0's output with device-to-device copies over NVLink while the next
step's convolution already runs (two local slabs and two output buffers in rotation; the timed region ends only when
the last copy has landed); `peer` -- the rank's kernel stores straight into rank 0's buffer (the assemble is the
kernel's own epilogue; its stores then wait on rank 0's link); `nccl` -- a local slab gathered with NCCL on the same
stream. Total work is fixed => "scaling": "strong".

A step = one full pass. `value` = GFLOP/s with slabs resident in HBM; `e2e` = the same pass from pinned host buffers
(H2D of the slab, conv, D2H of the result slab inside the timed region; the pass is cut along the batch dim so that the
upload of batch b+1, the convolution of batch b and the download of batch b-1 overlap on three streams). One JSON line
on stdout (rank 0).

`--impl reference` times the CPU implementation of the same path on the host cores (the oracle port; the JVM original
cannot run here). That arm never loads the CUDA library: inputs come from the host-only generator library.
"""
from __future__ import annotations

import argparse
import ctypes as C
import hashlib
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

A_SHAPE = [8, 32, 2048, 2048]
K_SHAPE = [1, 32, 5, 5]
SPLIT_DIM = 2


def shapes(scale: int):
    """--scale S divides the image's spatial extents by S (smoke / profiling runs); S = 1 is the real workload."""
    a = list(A_SHAPE)
    a[2] //= scale
    a[3] //= scale
    k = list(K_SHAPE)
    o = [abs(x - y) + 1 for x, y in zip(a, k)]
    return a, k, o


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Polls one GPU's SM clock, power and clock-event reasons through NVML (read-only) every few milliseconds while
    the timed region runs."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, gpu_index: int):
        self.rows, self.ok, self.stop_flag = [], False, False
        try:
            import pynvml
            self.nv = pynvml
            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            if vis:
                ids = [v.strip() for v in vis.split(",")]
                if gpu_index < len(ids) and ids[gpu_index].isdigit():
                    gpu_index = int(ids[gpu_index])
            self.h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.reason_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or pynvml.nvmlDeviceGetCurrentClocksThrottleReasons
            self.ok = True
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
        except Exception as e:  # no NVML: report that instead of clocks
            self.err = repr(e)

    def _poll(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                mask = self.reason_fn(self.h)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:
                    watts = None
                self.rows.append((time.time(), float(mhz), int(mask), watts))
            except Exception:
                pass
            time.sleep(0.002)

    def stop(self, t0: float, t1: float) -> dict:
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable: " + getattr(self, "err", "?")]}
        self.stop_flag = True
        self.thread.join(timeout=1.0)
        inside = [r for r in self.rows if t0 <= r[0] <= t1] or [r for r in self.rows if t0 - 0.01 <= r[0] <= t1 + 0.01]
        reasons = set()
        for r in inside:
            for bit, name in self.REASONS.items():
                if r[2] & bit:
                    reasons.add(name)
        watts = [r[3] for r in inside if r[3] is not None]
        return {"sm_mhz": float(np.median([r[1] for r in inside])) if inside else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(reasons), "samples": len(inside), "power_w_max": max(watts) if watts else None}


def kernel_traffic(kernel: str, workload: str):
    """DRAM bytes (read + write) of one launch of `kernel` on `workload`, as an ncu capture measured them -- from
    bench_traffic.json, and only while the kernel's source files still hash to what was captured (else None: a changed
    kernel has unknown traffic until it is captured again)."""
    path = os.path.join(ROOT, "bench_traffic.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        table = json.load(f)
    for row in table.get("captures", []):
        if row["workload"] == workload and kernel.startswith(row["kernel_prefix"]):
            h = hashlib.sha256()
            for rel in row["sources"]:
                with open(os.path.join(ROOT, rel), "rb") as src:
                    h.update(src.read())
            return float(row["dram_bytes_per_launch"]) if h.hexdigest() == row["sources_sha256"] else None
    return None


TRAFFIC_SOURCES = ["neureka_b200/csrc/nk_conv_tiled.cuh", "neureka_b200/csrc/nk_conv_tiled.cu"]


def record_traffic(dram_bytes: float, kernel_prefix: str, workload: str) -> None:
    """Writes a profiler-measured DRAM byte count into bench_traffic.json together with the hash of the kernel sources it
    was measured on (python bench.py --record-traffic BYTES, after reading dram__bytes_read.sum + dram__bytes_write.sum
    of one launch out of the capture)."""
    path = os.path.join(ROOT, "bench_traffic.json")
    table = {"captures": []}
    if os.path.exists(path):
        with open(path) as f:
            table = json.load(f)
    h = hashlib.sha256()
    for rel in TRAFFIC_SOURCES:
        with open(os.path.join(ROOT, rel), "rb") as src:
            h.update(src.read())
    table["captures"] = [r for r in table["captures"] if not (r["workload"] == workload and r["kernel_prefix"] == kernel_prefix)]
    table["captures"].append({"kernel_prefix": kernel_prefix, "workload": workload, "dram_bytes_per_launch": float(dram_bytes),
                              "sources": TRAFFIC_SOURCES, "sources_sha256": h.hexdigest()})
    with open(path, "w") as f:
        json.dump(table, f, indent=1)
        f.write("\n")


def bind_to_gpu_numa_node(gpu_index: int):
    """Runs this process on the CPUs of the NUMA node the GPU hangs off, so that the pinned staging buffers allocated
    afterwards are local to the GPU's PCIe root. Returns a short description, or why nothing was done."""
    try:
        import pynvml
        pynvml.nvmlInit()
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v.strip() for v in vis.split(",")]
            if gpu_index < len(ids) and ids[gpu_index].isdigit():
                gpu_index = int(ids[gpu_index])
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(gpu_index)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        bus = bus.lower()
        if len(bus.split(":")[0]) == 8:
            bus = bus[4:]
        handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            # the PCI device carries no node (virtualised topology): ask the driver which host memory nodes are closest
            try:
                n_nodes = len([d for d in os.listdir("/sys/devices/system/node") if d.startswith("node") and d[4:].isdigit()])
                words = pynvml.nvmlDeviceGetMemoryAffinity(handle, max(1, (n_nodes + 63) // 64), pynvml.NVML_AFFINITY_SCOPE_NODE)
                nodes = [i for i in range(n_nodes) if (words[i // 64] >> (i % 64)) & 1]
                if len(nodes) == 1 and n_nodes > 1:
                    node = nodes[0]
            except Exception:  # noqa: BLE001
                pass
        if node < 0:
            return "numa node unknown (-1)"
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return f"node {node}: none of its cpus allowed"
        os.sched_setaffinity(0, cpus)
        return f"node {node} ({len(cpus)} cpus)"
    except Exception as e:  # noqa: BLE001 -- placement is an optimisation, never a reason to fail
        return "not bound: " + repr(e)


def cpu_reference(seconds_target: float, reps: int = 1, gpu_out=None, k_shape=None, a_shape=None):
    """Times the CPU oracle (the line-faithful restatement of Neureka's CPU implementation) on a bounded sample of the
    benchmark's workload: the first rows of batch 0's output, computed from batch 0's 32 input planes, the flat output
    range split over all host threads like CPU.JVMExecutor splits it. Both arms of the benchmark call exactly this
    (same buffers -- ordinary numpy arrays it generates itself --, same calibration, same sample), so their figures are
    the same measurement. Returns a dict: best and mean GFLOP/s over `reps` repetitions, per-repetition values, cores,
    the sample's description and its share of the full pass, seconds per repetition, and the largest relative error
    of gpu_out (batch 0's output rows, if given) against the sample."""
    import baseline_configs as B
    from neureka_b200.ndconf import NDConfiguration as ND
    from oracle import oracle as O
    a_shape = a_shape or A_SHAPE
    k_shape = k_shape or K_SHAPE
    cores = os.cpu_count() or 1
    sa = [1, a_shape[1], a_shape[2], a_shape[3]]
    so = [1, 1, a_shape[2] - k_shape[2] + 1, a_shape[3] - k_shape[3] + 1]
    a_host = B.cfg5_image(n=int(np.prod(sa)))      # batch 0 = the first elements of the seed-5 stream
    k_host = B.cfg5_kernel()
    macs_per_out = k_shape[1] * k_shape[2] * k_shape[3]
    cfg_o, cfg_a, cfg_k = (ND.of_shape(s).as_inline_array() for s in (so, sa, k_shape))
    out = np.zeros(int(np.prod(so)), dtype=np.float32)
    row = so[3]

    def run(n_rows):
        n = n_rows * row
        chunk = (n + cores - 1) // cores
        ths = []
        t0 = time.perf_counter()
        for c in range(cores):
            s, e = c * chunk, min(n, (c + 1) * chunk)
            if s >= e:
                break
            th = threading.Thread(target=O.conv_range, args=(out, cfg_o, a_host, cfg_a, k_host, cfg_k, -1, s, e))
            th.start()
            ths.append(th)
        for th in ths:
            th.join()
        return time.perf_counter() - t0, n

    # calibrate on one row per thread (this also touches every page once), then size the sample for the target time
    t_cal, n_cal = run(min(cores, so[2]))
    rows = int(max(cores, min(so[2], seconds_target * (n_cal / t_cal) / row)))
    vals, secs = [], []
    for _ in range(max(1, reps)):
        t, n = run(rows)
        vals.append(2.0 * macs_per_out * n / t / 1e9)
        secs.append(t)
    err = None
    if gpu_out is not None:
        ref = out[:n].astype(np.float64)
        err = float(np.abs(gpu_out[:n].astype(np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))
    full_outputs = float(np.prod([a_shape[0], 1, so[2], so[3]]))
    return {"best": float(max(vals)), "mean": float(np.mean(vals)), "per_rep": [float(v) for v in vals], "cores": cores,
            "sample": f"first {rows} of {so[2]} output rows of batch 0 ({n} outputs x {macs_per_out} MACs)",
            "sample_fraction": n / full_outputs, "seconds_per_rep": [float(t) for t in secs], "max_rel_err": err}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--assemble", default="copy", choices=["copy", "peer", "nccl"])
    ap.add_argument("--scale", type=int, default=1)
    ap.add_argument("--conv-path", type=int, default=0, help="0 auto, 1 generic, 2 tiled, 3 tma")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--no-extra", action="store_true")
    ap.add_argument("--verify-assemble", action="store_true",
                    help="diagnostic (N > 1): rank 0 recomputes the whole convolution alone and compares the assembled "
                         "result bit for bit (adds 'assembled_equals_single_gpu' to the JSON line)")
    ap.add_argument("--probe-assemble", action="store_true",
                    help="diagnostic (N > 1, peer mode): time only the movement of the finished slabs into rank 0's "
                         "output (device-to-device copies over NVLink), i.e. the floor the owner's link sets for a step")
    ap.add_argument("--record-traffic", type=float, default=None,
                    help="no run: store this DRAM byte count (one full-size single-GPU launch, from a profiler capture) in "
                         "bench_traffic.json with the hash of the kernel's sources")
    args = ap.parse_args()
    if args.record_traffic is not None:
        record_traffic(args.record_traffic, "nk_conv_tiled_kernel<tma", "cfg5 full size, 1 GPU")
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    a_shape, k_shape, o_shape = shapes(args.scale)
    flops_total = 2.0 * np.prod(o_shape) * k_shape[1] * k_shape[2] * k_shape[3]
    config = {"workload": f"cfg5: F32 a{a_shape} x k{k_shape} -> {o_shape}, halo-split on dim {SPLIT_DIM}",
              "parallelism": f"slab{world}", "l2": "inputs larger than L2 (>= 512 MiB per GPU)"}

    # ------------------------------------------------------------------------------------------------------------
    # reference arm: the CPU implementation of the path on the host cores (the JVM original cannot run on this box;
    # the oracle is its line-faithful restatement). Nothing here loads the CUDA library.
    # ------------------------------------------------------------------------------------------------------------
    if args.impl == "reference":
        if rank != 0:
            return
        per = max(1.0, min(12.0, 150.0 / (steps + warmup)))
        r = cpu_reference(per, reps=warmup + steps, k_shape=k_shape, a_shape=a_shape)
        timed_vals = r["per_rep"][warmup:]
        timed_secs = r["seconds_per_rep"][warmup:]
        v = float(max(timed_vals))
        line = {"metric": "nd_conv_gflops", "value": v, "unit": "GFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
                "ms_per_step": 1e3 * float(np.mean(timed_secs)), "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f32", "data": "synthetic", "impl": "reference", "config": config,
                "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": r["cores"], "kind": "port",
                                 "sample": r["sample"] + " per step", "sample_fraction": r["sample_fraction"],
                                 "value_is": "best step", "mean": float(np.mean(timed_vals)), "per_step": timed_vals},
                "ms_per_step_is": "time of the sample that was computed, not of a full pass",
                "ms_full_pass_extrapolated": 1e3 * flops_total / (v * 1e9),
                "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    from neureka_b200 import _lib as L

    # ------------------------------------------------------------------------------------------------------------
    # CUDA arm
    # ------------------------------------------------------------------------------------------------------------
    from neureka_b200.device import CudaDevice
    from neureka_b200.ndconf import NDConfiguration as ND
    from neureka_b200.sharding import plan_slabs, slab_views

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group(backend="cpu:gloo,cuda:nccl")

    numa = bind_to_gpu_numa_node(local_rank)   # before any pinned allocation: staging memory local to the GPU's root
    dev = CudaDevice.get(local_rank)
    ctx = dev.ctx
    dev.set_conv_path(args.conv_path)

    ctx_copy = None   # second context (= second stream) of the `copy` assemble mode

    def barrier():
        dev.sync()
        if ctx_copy is not None:
            L.check(L.lib.nk_sync(ctx_copy), ctx_copy)
        if dist is not None:
            dist.barrier()

    halo = k_shape[SPLIT_DIM] - 1
    slab = plan_slabs(o_shape[SPLIT_DIM], world, halo)[rank]
    in_view, out_view, local_in_shape = slab_views(a_shape, k_shape, SPLIT_DIM, slab)
    local_out_shape = list(out_view.shape)
    n_in = int(np.prod(local_in_shape))
    n_out_local = int(np.prod(local_out_shape))
    n_out_full = int(np.prod(o_shape))

    # ---- synthetic inputs: java.util.Random streams, each rank generates only its slab -----------------------
    host_in = C.c_void_p()
    L.check(L.lib.nk_host_alloc(n_in * 4, C.byref(host_in)))
    host_out = C.c_void_p()
    L.check(L.lib.nk_host_alloc(max(n_out_local, 1) * 4, C.byref(host_out)))
    a_host = np.ctypeslib.as_array(C.cast(host_in, C.POINTER(C.c_float)), shape=(n_in,))
    out_host = np.ctypeslib.as_array(C.cast(host_out, C.POINTER(C.c_float)), shape=(max(n_out_local, 1),))
    plane = a_shape[2] * a_shape[3]
    seg = slab.in_len * a_shape[3]
    import baseline_configs as B
    for pl in range(a_shape[0] * a_shape[1]):
        B.cfg5_image(a_host[pl * seg:(pl + 1) * seg], start=pl * plane + slab.in_lo * a_shape[3])
    k_host = B.cfg5_kernel()

    def alloc(n, shared=False):
        """shared: from the plain allocator, so that the buffer can be exported to the other ranks"""
        b = C.c_void_p()
        L.check((L.lib.nk_alloc_shared if shared else L.lib.nk_alloc)(ctx, L.NK_F32, int(n), C.byref(b)), ctx)
        return b

    d_in, d_k, d_out_local = alloc(n_in), alloc(k_host.size), alloc(max(n_out_local, 1))
    L.check(L.lib.nk_write(ctx, d_in, host_in, 0, 0, n_in), ctx)
    L.check(L.lib.nk_write(ctx, d_k, k_host.ctypes.data_as(C.c_void_p), 0, 0, k_host.size), ctx)

    cfg_in = ND.of_shape(local_in_shape).as_inline_array()
    cfg_k = ND.of_shape(k_shape).as_inline_array()
    cfg_out_local = ND.of_shape(local_out_shape).as_inline_array()
    cfg_out_in_full = out_view.as_inline_array()
    pi = lambda arr: arr.ctypes.data_as(C.POINTER(C.c_int32))

    # ---- where the assembled result lives ----------------------------------------------------------------------
    d_full = None
    torch_full = torch_local = None
    if world == 1:
        d_full = d_out_local  # the slab is the whole output
    elif args.assemble == "copy":
        ctx_copy = C.c_void_p()
        L.check(L.lib.nk_device_open(local_rank, C.byref(ctx_copy)))
        handles = [(C.c_uint8 * L.NK_IPC_HANDLE_BYTES)() for _ in range(2)]
        d_fulls = []
        if rank == 0:
            for h in handles:
                d_fulls.append(alloc(n_out_full, shared=True))
                L.check(L.lib.nk_ipc_export(ctx, d_fulls[-1], h), ctx)
        box = [[bytes(h) for h in handles]]
        dist.broadcast_object_list(box, src=0)
        if rank != 0:
            for raw in box[0]:
                h = (C.c_uint8 * L.NK_IPC_HANDLE_BYTES).from_buffer_copy(raw)
                b = C.c_void_p()
                L.check(L.lib.nk_ipc_open(ctx, h, L.NK_F32, n_out_full, C.byref(b)), ctx)
                d_fulls.append(b)
        d_full = d_fulls[0]
        d_locals = [d_out_local, alloc(max(n_out_local, 1))]
        ev_conv, ev_copy = [], []
        for _ in range(2):
            for lst in (ev_conv, ev_copy):
                e = C.c_void_p()
                L.check(L.lib.nk_event_create(ctx, C.byref(e)), ctx)
                lst.append(e)
        step_no = [0]
    elif args.assemble == "peer":
        handle = (C.c_uint8 * L.NK_IPC_HANDLE_BYTES)()
        if rank == 0:
            d_full = alloc(n_out_full, shared=True)
            L.check(L.lib.nk_ipc_export(ctx, d_full, handle), ctx)
        box = [bytes(handle)]
        dist.broadcast_object_list(box, src=0)
        if rank != 0:
            h = (C.c_uint8 * L.NK_IPC_HANDLE_BYTES).from_buffer_copy(box[0])
            d_full = C.c_void_p()
            L.check(L.lib.nk_ipc_open(ctx, h, L.NK_F32, n_out_full, C.byref(d_full)), ctx)
    else:  # nccl: gather the local slabs on rank 0 through torch.distributed
        import torch
        ptr = C.c_void_p(); L.lib.nk_buf_info(d_out_local, C.byref(ptr), None, None)
        stream = torch.cuda.ExternalStream(L.lib.nk_stream(ctx))
        torch.cuda.set_stream(stream)
        # NCCL gather wants equal sizes: every rank contributes a buffer of the largest slab's size
        sizes = [int(np.prod(slab_views(a_shape, k_shape, SPLIT_DIM, s)[1].shape)) for s in plan_slabs(o_shape[SPLIT_DIM], world, halo)]
        n_pad = max(sizes)
        torch_local = torch.empty(n_pad, dtype=torch.float32, device=f"cuda:{local_rank}")
        wrapped = C.c_void_p()
        L.check(L.lib.nk_wrap(ctx, L.NK_F32, C.c_void_p(torch_local.data_ptr()), n_pad, C.byref(wrapped)), ctx)
        d_out_nccl = wrapped
        gather_list = [torch.empty(n_pad, dtype=torch.float32, device=f"cuda:{local_rank}") for _ in sizes] if rank == 0 else None

    def conv_step_resident():
        """One pass with slabs resident: conv into the assembled output (peer stores) or local slab (+ NCCL gather)."""
        if n_out_local == 0:
            return
        if world == 1:
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_out_local, pi(cfg_out_local), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
        elif args.assemble == "copy":
            j = step_no[0] % 2
            step_no[0] += 1
            if rank == 0:   # the owner computes straight into place
                L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_fulls[j], pi(cfg_out_in_full), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
                return
            L.check(L.lib.nk_stream_wait_event(ctx, ev_copy[j]), ctx)        # the push that last read this local slab is done
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_locals[j], pi(cfg_out_local), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
            L.check(L.lib.nk_event_record(ctx, ev_conv[j]), ctx)
            L.check(L.lib.nk_stream_wait_event(ctx_copy, ev_conv[j]), ctx_copy)
            rows = local_out_shape[2] * local_out_shape[3]
            full_rows = o_shape[2] * o_shape[3]
            for b in range(o_shape[0] * o_shape[1]):
                L.check(L.lib.nk_copy(ctx_copy, d_fulls[j], b * full_rows + slab.out_lo * o_shape[3], d_locals[j], b * rows, rows), ctx_copy)
            L.check(L.lib.nk_event_record(ctx_copy, ev_copy[j]), ctx_copy)
        elif args.assemble == "peer":
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_full, pi(cfg_out_in_full), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
        else:
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_out_nccl, pi(cfg_out_local), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
            dist.gather(torch_local, gather_list, dst=0)

    def assemble_only_step():
        """Copies of this rank's finished slab into its place in rank 0's output, one per outer index (contiguous rows)."""
        if n_out_local == 0 or rank == 0:
            return
        rows = local_out_shape[2] * local_out_shape[3]
        full_rows = o_shape[2] * o_shape[3]
        for b in range(o_shape[0] * o_shape[1]):
            L.check(L.lib.nk_copy(ctx, d_full, b * full_rows + slab.out_lo * o_shape[3], d_out_local, b * rows, rows), ctx)

    # ---- the pass from host buffers, cut along the batch dim: upload of batch b+1 | convolution of batch b | download
    # of batch b-1 on three streams (each context owns one), ordered by events. The local slab is dense
    # [batches, channels, rows, width], so a batch is one contiguous range on either side.
    e2e = {}

    def e2e_setup():
        nb = local_in_shape[0]
        e2e["nb"] = nb
        e2e["in_per"] = n_in // nb
        e2e["out_per"] = n_out_local // nb
        for name in ("ctx_up", "ctx_down"):
            c = C.c_void_p()
            L.check(L.lib.nk_device_open(local_rank, C.byref(c)))
            e2e[name] = c
        for name in ("up", "conv"):
            evs = []
            for _ in range(nb):
                ev = C.c_void_p()
                L.check(L.lib.nk_event_create(ctx, C.byref(ev)), ctx)
                evs.append(ev)
            e2e["ev_" + name] = evs
        ev = C.c_void_p()
        L.check(L.lib.nk_event_create(ctx, C.byref(ev)), ctx)
        e2e["ev_done"] = ev
        sh_in = [1] + list(local_in_shape[1:])
        sh_out = [1] + list(local_out_shape[1:])
        e2e["cfg_in"] = [ND.of_shape(local_in_shape).sliced(sh_in, [b, 0, 0, 0], [1, 1, 1, 1]).as_inline_array() for b in range(nb)]
        e2e["cfg_out"] = [ND.of_shape(local_out_shape).sliced(sh_out, [b, 0, 0, 0], [1, 1, 1, 1]).as_inline_array() for b in range(nb)]

    def conv_step_e2e():
        """The same pass from host buffers: H2D of the slab, conv, D2H of the rank's result slab, batch by batch."""
        if n_out_local == 0:
            return
        up, down = e2e["ctx_up"], e2e["ctx_down"]
        ip, op = e2e["in_per"], e2e["out_per"]
        L.check(L.lib.nk_stream_wait_event(up, e2e["ev_done"]), up)        # the previous pass has read d_in completely
        for b in range(e2e["nb"]):
            L.check(L.lib.nk_write_async(up, d_in, host_in, b * ip, b * ip, ip), up)
            L.check(L.lib.nk_event_record(up, e2e["ev_up"][b]), up)
            L.check(L.lib.nk_stream_wait_event(ctx, e2e["ev_up"][b]), ctx)
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_out_local, pi(e2e["cfg_out"][b]), d_in, pi(e2e["cfg_in"][b]), d_k, pi(cfg_k), -1), ctx)
            L.check(L.lib.nk_event_record(ctx, e2e["ev_conv"][b]), ctx)
            L.check(L.lib.nk_stream_wait_event(down, e2e["ev_conv"][b]), down)
            L.check(L.lib.nk_read_async(down, d_out_local, C.c_void_p(host_out.value + b * op * 4), b * op, op), down)
        L.check(L.lib.nk_event_record(down, e2e["ev_done"]), down)
        L.check(L.lib.nk_stream_wait_event(ctx, e2e["ev_done"]), ctx)       # the launch stream's timer sees the whole pass

    def timed(fn, n_warm, n_steps):
        """W untimed steps, then exactly K steps between two events on the launch stream, bracketed by barrier +
        synchronise on both sides; returns (max-over-ranks ms, wall t0, wall t1, kernels this rank launched)."""
        for _ in range(n_warm):
            fn()
        barrier()
        n0 = dev.launch_count()
        t0 = time.time()
        L.check(L.lib.nk_timer_begin(ctx), ctx)
        for _ in range(n_steps):
            fn()
        if world > 1 and args.assemble == "copy" and rank != 0:
            for e in ev_copy:   # the timed region ends when the last pushes have landed in rank 0's memory
                L.check(L.lib.nk_stream_wait_event(ctx, e), ctx)
        ms = C.c_float(0)
        L.check(L.lib.nk_timer_end(ctx, C.byref(ms)), ctx)   # records the end event and synchronises on it
        barrier()
        t1 = time.time()
        n1 = dev.launch_count()
        m = float(ms.value)
        if dist is not None:
            import torch
            t = torch.tensor([m], dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            m = float(t.item())
        return m, t0, t1, n1 - n0

    if args.probe_assemble:
        if world == 1 or args.assemble == "nccl":
            raise SystemExit("--probe-assemble needs N > 1 and --assemble copy or peer")
        ms_total, _, _, _ = timed(assemble_only_step, max(warmup, 3), steps)
        if rank == 0:
            moved = (n_out_full - n_out_local) * 4
            print(json.dumps({"probe": "assemble_only", "n_gpus": world, "ms_per_step": ms_total / steps, "bytes_into_rank0": moved,
                              "gbs_into_rank0": moved / (ms_total / steps * 1e-3) / 1e9}))
        barrier()
        dist.destroy_process_group()
        return
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms_total, t0, t1, launches = timed(conv_step_resident, max(warmup, 3), steps)
    clocks = sampler.stop(t0, t1) if sampler else None
    last_kernel = dev.last_kernel()
    conv_family = dev.last_conv_path()
    ms_step = ms_total / steps
    value = flops_total / (ms_step * 1e-3) / 1e9

    # one pass alone, start to assembled result, nothing of a neighbouring pass overlapping it (median of 7)
    single_pass_ms = None
    if world > 1:
        singles = []
        for _ in range(7):
            m, _, _, _ = timed(conv_step_resident, 0, 1)
            singles.append(m)
        single_pass_ms = float(np.median(singles))

    e2e_setup()
    n_e2e = max(2, min(steps, 5))
    e2e_ms_total, _, _, _ = timed(conv_step_e2e, 1, n_e2e)
    e2e_ms = e2e_ms_total / n_e2e
    e2e_value = flops_total / (e2e_ms * 1e-3) / 1e9
    h2d = n_in * 4
    d2h = n_out_local * 4
    e2e_ok = None
    if world == 1:   # the pipelined pass must leave the same result in the host buffer as the resident pass left on the device
        L.check(L.lib.nk_sync(e2e["ctx_down"]), e2e["ctx_down"])
        check = np.empty(n_out_local, dtype=np.float32)
        L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_out_local, pi(cfg_out_local), d_in, pi(cfg_in), d_k, pi(cfg_k), -1), ctx)
        L.check(L.lib.nk_read(ctx, d_out_local, check.ctypes.data_as(C.c_void_p), 0, n_out_local), ctx)
        e2e_ok = bool(np.array_equal(check, out_host[:n_out_local]))
    if dist is not None:
        import torch
        t = torch.tensor([h2d, d2h, launches], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        h2d, d2h, launches = int(t[0].item()), int(t[1].item()), int(t[2].item())

    assembled_ok = None
    if args.verify_assemble and world > 1:
        barrier()
        if rank == 0:
            n_full_in = int(np.prod(a_shape))
            full_host = B.cfg5_image(n=n_full_in)
            d_a, d_ref = alloc(n_full_in), alloc(n_out_full)
            L.check(L.lib.nk_write(ctx, d_a, full_host.ctypes.data_as(C.c_void_p), 0, 0, n_full_in), ctx)
            cfg_a, cfg_o = ND.of_shape(a_shape).as_inline_array(), ND.of_shape(o_shape).as_inline_array()
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_ref, pi(cfg_o), d_a, pi(cfg_a), d_k, pi(cfg_k), -1), ctx)
            want = np.empty(n_out_full, dtype=np.float32)
            L.check(L.lib.nk_read(ctx, d_ref, want.ctypes.data_as(C.c_void_p), 0, n_out_full), ctx)
            got = np.empty(n_out_full, dtype=np.float32)
            assembled_ok = True
            if args.assemble == "nccl":
                sl = plan_slabs(o_shape[SPLIT_DIM], world, halo)
                w4 = want.reshape(o_shape)
                for g, t in enumerate(gather_list):
                    sh = list(o_shape); sh[SPLIT_DIM] = sl[g].out_len
                    part = t[: int(np.prod(sh))].cpu().numpy().reshape(sh)
                    assembled_ok = assembled_ok and bool(np.array_equal(part, w4[:, :, sl[g].out_lo:sl[g].out_hi, :]))
            else:
                for buf in (d_fulls if args.assemble == "copy" else [d_full]):
                    L.check(L.lib.nk_read(ctx, buf, got.ctypes.data_as(C.c_void_p), 0, n_out_full), ctx)
                    assembled_ok = assembled_ok and bool(np.array_equal(got, want))
            L.lib.nk_free(ctx, d_a); L.lib.nk_free(ctx, d_ref)
        barrier()

    sharded = None
    if world > 1 and not args.no_extra:   # collectives inside: every rank takes part
        from bench_sharded import run_sharded_extra
        sharded = run_sharded_extra(dev, dist, rank, world, local_rank, read_peaks()[0])

    if rank == 0:
        peak, peak_kind = read_peaks()
        # algorithmic bytes of rank 0's launch: its input slab + the kernel + its output slab, each touched once
        alg_bytes = (n_in + k_host.size + n_out_local) * 4.0
        alg_flops = 2.0 * n_out_local * k_shape[1] * k_shape[2] * k_shape[3]
        kernel_ms = ms_step  # one conv kernel per step on this rank
        achieved = alg_bytes / (kernel_ms * 1e-3) / 1e9
        # DRAM bytes (read + write) of one launch, from the profiler capture of this very launch shape (None when the
        # kernel's sources changed since, or for sizes that were not captured)
        traffic = kernel_traffic(last_kernel, "cfg5 full size, 1 GPU") if (world == 1 and args.scale == 1) else None
        props = dev.props
        fma_nominal = props.sm_count * 128 * 2 * props.clock_khz * 1e3 / 1e12   # FP32 lanes per SM x 2 flop x clock
        roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                    "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
                    "kernel": last_kernel, "kernel_ms": kernel_ms, "algorithmic_bytes_per_launch": alg_bytes,
                    "fp32_fma": {"achieved_tflops": alg_flops / (kernel_ms * 1e-3) / 1e12, "nominal_peak_tflops": fma_nominal}}
        line = {"metric": "nd_conv_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": steps, "warmup": max(warmup, 3),
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config, "conv_family": conv_family,
                "e2e": {"value": e2e_value, "unit": "GFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                        "pipeline": "per batch: upload | convolution | download on three streams", "staging_numa": numa,
                        "h2d_gbs_per_gpu": (h2d / world) / (e2e_ms * 1e-3) / 1e9, "matches_resident_result": e2e_ok},
                "gpu_launches": int(launches), "roofline": roofline, "clocks": clocks}
        if world > 1:
            line["assemble"] = {"mode": args.assemble,
                                "overlap": ("the push of pass k into rank 0's output runs on a second stream under the convolution of pass k+1; "
                                            "ms_per_step is therefore a pipelined throughput figure, every push inside the timed region")
                                if args.assemble == "copy" else "none: a pass is assembled when its kernel (or gather) retires",
                                "single_pass_ms": single_pass_ms}
        if world == 1:
            # CPU baseline on a bounded sample of the same workload (the routine the reference arm runs), checked against
            # the GPU result on the way
            L.check(L.lib.nk_read(ctx, d_out_local, host_out, 0, n_out_local), ctx)
            r = cpu_reference(args.cpu_seconds / 2, reps=2, gpu_out=out_host, k_shape=k_shape, a_shape=a_shape)
            line["cpu_baseline"] = {"value": r["best"], "unit": "GFLOP/s", "cores": r["cores"], "kind": "port", "sample": r["sample"],
                                    "sample_fraction": r["sample_fraction"], "value_is": "best of 2 repetitions", "per_rep": r["per_rep"],
                                    "gpu_vs_cpu_max_rel_err_on_sample": r["max_rel_err"]}
            if not args.no_extra:
                try:
                    from bench_extra import run_extra
                    line["extra"] = run_extra(dev, peak)
                    fp32 = line["extra"]["measured_fma_peak_tflops"]["fp32"]
                    roofline["fp32_fma"]["measured_peak_tflops"] = fp32
                    roofline["fp32_fma"]["frac_of_measured"] = roofline["fp32_fma"]["achieved_tflops"] / fp32
                except Exception as e:  # the headline line must survive a failing side measurement
                    line["extra"] = {"error": repr(e)}
        if assembled_ok is not None:
            line["assembled_equals_single_gpu"] = assembled_ok
        if sharded is not None:
            line["extra"] = {"sharded": sharded}
        print(json.dumps(line))
        sys.stdout.flush()

    barrier()
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
