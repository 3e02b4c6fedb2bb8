"""Side measurements of the sharded paths beside the forward convolution, for `bench.py` runs with N > 1
(reported under `extra` of the JSON line; one process per GPU, launched by torchrun):

* BASELINE config 3 -- `tanh(a*b + b)` with a [4096,1,1024], b [1,2048,1024] and the gradients of its sum -- split along
  dim 0 of `a` (rows of the output): no communication forward; the gradient of `a` is local; the gradient of `b` is a
  sum over the split dim, so every rank reduces its rows and the 8 MiB partials meet in one NCCL all-reduce.
* The two gradients of BASELINE config 5's convolution under the same halo split as the forward pass: the image
  gradient shards like the forward with the halo on the *error* side (a rank's rows need the error rows from 4 above);
  the kernel gradient (800 values) is a full reduction: per-rank partials + one tiny all-reduce.

Every timed region is bracketed by barrier + synchronise, device-timed with events, max over ranks.

Keeping the ranks in step when one of them fails. A stage has two kinds of code. *Local* work (allocations, uploads,
kernel launches, host checks) can fail on one rank alone -- out of memory, a refused argument. *Collectives* must be
entered by every rank or by none: a rank that skipped one would leave its peers spinning inside it on their GPUs. So
(1) everything a stage allocates is prepared before its first collective, then the ranks agree over the CPU (gloo)
group whether all of them succeeded and skip the stage together if not; (2) after that point local work runs through
`_Guard.local`, which records an exception instead of raising it, so the rank still enters every collective of the
stage; (3) at the end the ranks agree again and report the error together.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

import baseline_configs as B
from neureka_b200 import _lib as L
from neureka_b200 import jrand
from neureka_b200.ndconf import NDConfiguration as ND
from neureka_b200.sharding import plan_image_grad_slabs, plan_slabs


class StageSkipped(Exception):
    """Some rank failed before the stage's first collective; every rank leaves the stage here."""


def agree(dist, ok: bool) -> bool:
    """True when every rank says ok. A CPU all-reduce (gloo): it does not touch the GPUs' streams."""
    import torch
    t = torch.tensor([1 if ok else 0], dtype=torch.int32)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return bool(t.item() == 1)


class _Guard:
    """Runs local work of a stage whose collectives have begun: the first exception is kept, later local work is
    skipped, and the caller goes on to the next collective like every other rank."""

    def __init__(self):
        self.error = None

    def local(self, fn, default=None):
        if self.error is not None:
            return default
        try:
            return fn()
        except Exception as e:   # noqa: BLE001 -- reported by the stage, after the ranks agreed
            self.error = e
            return default


def _cfg(conf_or_shape):
    c = conf_or_shape if isinstance(conf_or_shape, ND) else ND.of_shape(conf_or_shape)
    a = c.as_inline_array()
    return a, a.ctypes.data_as(C.POINTER(C.c_int32))


def _alloc(ctx, n, dt=L.NK_F32):
    b = C.c_void_p()
    L.check(L.lib.nk_alloc(ctx, dt, int(n), C.byref(b)), ctx)
    return b


def _upload(ctx, buf, host):
    h = np.ascontiguousarray(host)
    L.check(L.lib.nk_write(ctx, buf, h.ctypes.data_as(C.c_void_p), 0, 0, h.size), ctx)


def _download(ctx, buf, n, dtype=np.float32, start=0):
    out = np.empty(int(n), dtype=dtype)
    L.check(L.lib.nk_read(ctx, buf, out.ctypes.data_as(C.c_void_p), int(start), int(n)), ctx)
    return out


def _rand(n, dist_kind, seed, p0, p1, start=0):
    return jrand.fill(np.empty(int(n), dtype=np.float32), dist_kind, seed, p0, p1, int(start))


class _Timer:
    """K launches of `fn` between two events, bracketed by barrier + synchronise; max over ranks. `fn` must not raise
    (local work inside it goes through a _Guard) so that every rank enters the same collectives."""

    def __init__(self, dev, dist):
        self.dev, self.dist, self.ctx = dev, dist, dev.ctx

    def barrier(self):
        try:
            self.dev.sync()
        except Exception:   # noqa: BLE001 -- a failed stream shows up in the stage's guard; the barrier must still be met
            pass
        self.dist.barrier()

    def __call__(self, fn, warm=2, reps=5):
        import torch
        for _ in range(warm):
            fn()
        self.barrier()
        L.lib.nk_timer_begin(self.ctx)
        for _ in range(reps):
            fn()
        ms = C.c_float(0)
        L.lib.nk_timer_end(self.ctx, C.byref(ms))
        self.barrier()
        t = torch.tensor([float(ms.value) / reps], dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def _torch_view_of(ctx, local_rank, n):
    """A torch tensor and an nk_buf over the same device memory, for collectives on the context's stream."""
    import torch
    t = torch.empty(int(n), dtype=torch.float32, device=f"cuda:{local_rank}")
    b = C.c_void_p()
    L.check(L.lib.nk_wrap(ctx, L.NK_F32, C.c_void_p(t.data_ptr()), int(n), C.byref(b)), ctx)
    return t, b


def _prepared(dist, prepare):
    """Runs the local set-up of a stage, then lets the ranks agree: returns its result, or raises StageSkipped on
    every rank when any rank failed (the failing rank's own message goes into the exception)."""
    state, err = None, None
    try:
        state = prepare()
    except Exception as e:   # noqa: BLE001
        err = e
    if not agree(dist, err is None):
        raise StageSkipped(repr(err) if err is not None else "another rank failed while preparing this stage")
    return state


def broadcast_sharded(dev, dist, rank, world, local_rank, hbm_peak_gbs):
    import torch
    ctx = dev.ctx
    n, m, k = 4096, 2048, 1024
    if n % world:
        return {"skipped": f"4096 rows do not split evenly over {world} ranks"}
    rows = n // world
    N = rows * m * k                                    # outputs of this rank
    bufs = []

    def prepare():
        if dev.props.total_mem_bytes < 3 * N * 4 + (8 << 30):
            raise MemoryError("not enough device memory for three slab-sized intermediates")
        torch.cuda.set_stream(torch.cuda.ExternalStream(L.lib.nk_stream(ctx)))
        # one uniform stream of seed 3: a (this rank's rows of it), then b
        a_h = _rand(rows * k, 0, 3, -2.0, 2.0, start=rank * rows * k)
        b_h = _rand(m * k, 0, 3, -2.0, 2.0, start=n * k)
        for cnt in (rows * k, m * k, rows * k, N, N, N, rows * k):
            bufs.append(_alloc(ctx, cnt))
        a, b = bufs[0], bufs[1]
        _upload(ctx, a, a_h); _upload(ctx, b, b_h)
        gb_t, gb = _torch_view_of(ctx, local_rank, m * k)
        bufs.append(gb)
        return a_h, b_h, gb_t

    try:
        a_h, b_h, gb_t = _prepared(dist, prepare)
    except StageSkipped:
        for buf in bufs:
            L.lib.nk_free(ctx, buf)
        raise
    a, b, a1, t, y, g, ga, gb = bufs
    ca, pa = _cfg([rows, 1, k]); cb, pb = _cfg([1, m, k]); co, po = _cfg([rows, m, k])
    guard = _Guard()

    def forward():
        def launches():
            L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t, po, a, pa, b, pb, -1), ctx)
            L.check(L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, y, po, t, po, b, pb, -1), ctx)
            L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, t, po, y, po, -1), ctx)
        guard.local(launches)

    def backward():
        # error of sum(tanh(...)) is all ones: g = tanh'(y); da = sum_j g*b; db = sum_i g*(a+1), then the ranks' partials meet
        def launches():
            L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g, po, y, po, 0), ctx)
            L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga, pa, b, pb, g, po, 0), ctx)
            L.check(L.lib.nk_scalar_binary(ctx, L.NK_OP_ADD, L.NK_F32, 3, a1, pa, a, pa, 1.0, -1), ctx)
            L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, gb, pb, a1, pa, g, po, 0), ctx)
        guard.local(launches)
        dist.all_reduce(gb_t, op=dist.ReduceOp.SUM)

    timer = _Timer(dev, dist)
    fwd_ms = timer(forward, 1, 3)
    bwd_ms = timer(backward, 1, 3)

    def spot_check():
        # a window of the forward result on this rank against float64 numpy, and the summed gradient finite
        win = 2048
        got = _download(ctx, t, win, start=N - win)
        idx = np.arange(N - win, N, dtype=np.int64)
        i, j, kk = idx // (m * k), (idx // k) % m, idx % k
        u = (a_h[i * k + kk] * b_h[j * k + kk]).astype(np.float32) + b_h[j * k + kk]
        ok_fwd = bool(np.abs(got - np.tanh(u.astype(np.float64))).max() <= 2e-7 * 4)
        gb_all = _download(ctx, gb, m * k)
        return [1.0 if ok_fwd else 0.0, float(np.isfinite(gb_all).all())]

    flags = torch.tensor(guard.local(spot_check, [0.0, 0.0]), dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    for buf in bufs:
        L.lib.nk_free(ctx, buf)
    if not agree(dist, guard.error is None):
        return {"error": repr(guard.error) if guard.error is not None else "another rank failed in this stage"}
    fwd_bytes = world * 4.0 * ((N + rows * k + m * k) + (2 * N + m * k) + 2 * N)
    bwd_bytes = world * 4.0 * (2 * N + (N + rows * k + m * k) * 2)
    return {"n_gpus": world, "rows_per_gpu": rows, "outputs_total": world * N,
            "forward_ms": fwd_ms, "forward_gbs_total": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
            "backward_ms": bwd_ms, "backward_gbs_total": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
            "frac_of_hbm_peak_forward": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / (world * hbm_peak_gbs),
            "frac_of_hbm_peak_backward": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / (world * hbm_peak_gbs),
            "collective": "one NCCL all-reduce of the 8 MiB partial gradient of b per backward pass",
            "forward_window_matches_numpy": bool(flags[0].item() == 1.0), "gradient_finite": bool(flags[1].item() == 1.0),
            "note": "forward = mul-broadcast, add-broadcast, tanh (op by op, as the reference evaluates it)"}


def xconv_sharded(dev, dist, rank, world, local_rank, scale=1):
    """Image gradient and kernel gradient of config 5 under the forward pass's row split. With scale > 1 (smaller
    image) rank 0 also recomputes both gradients alone and compares."""
    import torch
    ctx = dev.ctx
    Bn, Cn, H, W, KH = 8, 32, 2048 // scale, 2048 // scale, 5
    OH, OW = H - KH + 1, W - KH + 1
    halo = KH - 1
    # image-gradient rows [lo, hi) of the H image rows; error rows needed: [lo - halo, hi) clipped to [0, OH)
    gs = plan_image_grad_slabs(H, world, halo)[rank]
    lo, hi, e_lo = gs.lo, gs.hi, gs.err_lo
    re = gs.err_len                                    # error rows held for the image gradient
    # kernel gradient: this rank's error rows [f_lo, f_hi) of the forward split and image rows [f_lo, f_hi + halo)
    f = plan_slabs(OH, world, halo)[rank]
    rf = f.out_len
    bufs = []

    def prepare():
        torch.cuda.set_stream(torch.cuda.ExternalStream(L.lib.nk_stream(ctx)))
        k_h = B.cfg5_kernel()
        err_rows = np.empty((Bn, re, OW), dtype=np.float32)
        for b in range(Bn):
            err_rows[b] = _rand(re * OW, 0, 9, -1.0, 1.0, start=b * OH * OW + e_lo * OW).reshape(re, OW)
        img = np.empty((Bn * Cn, f.in_len, W), dtype=np.float32)
        for pl in range(Bn * Cn):
            img[pl] = _rand(f.in_len * W, 0, 5, 0.0, 1.0, start=pl * H * W + f.in_lo * W).reshape(f.in_len, W)
        err_f = np.empty((Bn, rf, OW), dtype=np.float32)
        for b in range(Bn):
            err_f[b] = _rand(rf * OW, 0, 9, -1.0, 1.0, start=b * OH * OW + f.out_lo * OW).reshape(rf, OW)
        # local drain of the deconvolution: re + halo rows; rows [lo - e_lo, lo - e_lo + (hi - lo)) of it are this rank's
        for cnt in (k_h.size, Bn * re * OW, Bn * Cn * (re + halo) * W, img.size, err_f.size):
            bufs.append(_alloc(ctx, cnt))
        _upload(ctx, bufs[0], k_h); _upload(ctx, bufs[1], err_rows); _upload(ctx, bufs[3], img); _upload(ctx, bufs[4], err_f)
        gk_t, d_gk = _torch_view_of(ctx, local_rank, Cn * KH * KH)
        bufs.append(d_gk)
        return gk_t

    try:
        gk_t = _prepared(dist, prepare)
    except StageSkipped:
        for buf in bufs:
            L.lib.nk_free(ctx, buf)
        raise
    d_k, d_e, d_ga, d_img, d_ef, d_gk = bufs
    c_ga, p_ga = _cfg([Bn, Cn, re + halo, W]); c_k, p_k = _cfg([1, Cn, KH, KH]); c_e, p_e = _cfg([Bn, 1, re, OW])
    c_img, p_img = _cfg([Bn, Cn, f.in_len, W]); c_ef, p_ef = _cfg([Bn, 1, rf, OW])
    guard = _Guard()

    def grad_image():
        guard.local(lambda: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_ga, p_ga, d_k, p_k, d_e, p_e, 0), ctx))

    def grad_kernel():
        guard.local(lambda: L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_gk, p_k, d_img, p_img, d_ef, p_ef, 0), ctx))
        dist.all_reduce(gk_t, op=dist.ReduceOp.SUM)

    timer = _Timer(dev, dist)
    ga_ms = timer(grad_image, 2, 10)
    ga_kernel = dev.last_kernel()
    gk_ms = timer(grad_kernel, 2, 10)
    gk_kernel = dev.last_kernel()
    flops = 2.0 * Bn * OH * OW * Cn * KH * KH
    out = {"n_gpus": world, "image": [Bn, Cn, H, W], "grad_image_ms": ga_ms, "grad_image_tflops_total": flops / (ga_ms * 1e-3) / 1e12,
           "grad_image_kernel": ga_kernel, "grad_kernel_ms": gk_ms, "grad_kernel_tflops_total": flops / (gk_ms * 1e-3) / 1e12,
           "grad_kernel_kernel": gk_kernel,
           "split": "rows of the image gradient / of the error; error halo of 4 rows above; kernel gradient = partials + all-reduce of 800 values"}

    if scale > 1:
        # gather the ranks' rows on rank 0 (host side, small) and compare with a single-GPU computation of the whole thing
        grad_image(); grad_kernel()

        def my_rows():
            dev.sync()
            return _download(ctx, d_ga, Bn * Cn * (re + halo) * W).reshape(Bn, Cn, re + halo, W)[:, :, lo - e_lo: lo - e_lo + (hi - lo), :]

        mine = guard.local(my_rows)
        parts = [None] * world
        dist.all_gather_object(parts, mine)

        def compare_on_rank0():
            gk = _download(ctx, d_gk, Cn * KH * KH)
            if any(p is None for p in parts):
                raise RuntimeError("a rank delivered no gradient rows")
            full_e = np.empty((Bn, OH, OW), dtype=np.float32)
            for b in range(Bn):
                full_e[b] = _rand(OH * OW, 0, 9, -1.0, 1.0, start=b * OH * OW).reshape(OH, OW)
            full_a = _rand(Bn * Cn * H * W, 0, 5, 0.0, 1.0)
            tmp = []
            try:
                for cnt in (full_e.size, full_a.size, Bn * Cn * H * W, Cn * KH * KH):
                    tmp.append(_alloc(ctx, cnt))
                dE, dA, dGA, dGK = tmp
                _upload(ctx, dE, full_e); _upload(ctx, dA, full_a)
                cA, pA = _cfg([Bn, Cn, H, W]); cE, pE = _cfg([Bn, 1, OH, OW])
                L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, dGA, pA, d_k, p_k, dE, pE, 0), ctx)
                L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, dGK, p_k, dA, pA, dE, pE, 0), ctx)
                want_a = _download(ctx, dGA, Bn * Cn * H * W).reshape(Bn, Cn, H, W)
                want_k = _download(ctx, dGK, Cn * KH * KH)
            finally:
                for buf in tmp:
                    L.lib.nk_free(ctx, buf)
            got_a = np.concatenate(parts, axis=2)
            out["grad_image_equals_single_gpu"] = bool(np.array_equal(got_a, want_a))
            out["grad_kernel_rel_err_vs_single_gpu"] = float(np.abs(gk - want_k).max() / np.abs(want_k).max())

        if rank == 0:
            guard.local(compare_on_rank0)
        dist.barrier()
    for buf in bufs:
        L.lib.nk_free(ctx, buf)
    if not agree(dist, guard.error is None):
        return {"error": repr(guard.error) if guard.error is not None else "another rank failed in this stage"}
    return out


def run_sharded_extra(dev, dist, rank, world, local_rank, hbm_peak_gbs):
    out = {}
    for name, fn in (("cfg5_gradients_sharded_check_scale4", lambda: xconv_sharded(dev, dist, rank, world, local_rank, scale=4)),
                     ("cfg5_gradients_sharded", lambda: xconv_sharded(dev, dist, rank, world, local_rank, scale=1)),
                     ("cfg3_sharded_rows", lambda: broadcast_sharded(dev, dist, rank, world, local_rank, hbm_peak_gbs))):
        try:
            out[name] = fn()
        except StageSkipped as e:   # agreed by all ranks before the stage's first collective: all of them are here
            out[name] = {"skipped": str(e)}
    return out
