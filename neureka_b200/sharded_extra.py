"""Side measurements of the sharded paths beside the forward convolution, for `bench.py` runs with N > 1
(reported under `extra` of the JSON line; one process per GPU, launched by torchrun):

* BASELINE config 3 -- `tanh(a*b + b)` with a [4096,1,1024], b [1,2048,1024] and the gradients of its sum -- split along
  dim 0 of `a` (rows of the output): no communication forward; the gradient of `a` is local; the gradient of `b` is a
  sum over the split dim, so every rank reduces its rows and the 8 MiB partials meet in one NCCL all-reduce.
* The two gradients of BASELINE config 5's convolution under the same halo split as the forward pass: the image
  gradient shards like the forward with the halo on the *error* side (a rank's rows need the error rows from 4 above);
  the kernel gradient (800 values) is a full reduction: per-rank partials + one tiny all-reduce.

Every timed region is bracketed by barrier + synchronise, device-timed with events, max over ranks.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib as L
from .ndconf import NDConfiguration as ND
from .sharding import plan_image_grad_slabs, plan_slabs


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
    a = np.empty(int(n), dtype=np.float32)
    L.lib.nk_jrand_fill_at(L.NK_F32, dist_kind, seed, p0, p1, int(start), a.ctypes.data_as(C.c_void_p), int(n))
    return a


class _Timer:
    def __init__(self, dev, dist):
        self.dev, self.dist, self.ctx = dev, dist, dev.ctx

    def barrier(self):
        self.dev.sync()
        self.dist.barrier()

    def __call__(self, fn, warm=2, reps=5):
        import torch
        for _ in range(warm):
            fn()
        self.barrier()
        L.check(L.lib.nk_timer_begin(self.ctx), self.ctx)
        for _ in range(reps):
            fn()
        ms = C.c_float(0)
        L.check(L.lib.nk_timer_end(self.ctx, C.byref(ms)), self.ctx)
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


def broadcast_sharded(dev, dist, rank, world, local_rank, hbm_peak_gbs):
    import torch
    ctx = dev.ctx
    n, m, k = 4096, 2048, 1024
    if n % world:
        return {"skipped": f"4096 rows do not split evenly over {world} ranks"}
    rows = n // world
    N = rows * m * k                                    # outputs of this rank
    need = 3 * N * 4
    if dev.props.total_mem_bytes < need + (8 << 30):
        return {"skipped": "not enough device memory for three slab-sized intermediates"}
    torch.cuda.set_stream(torch.cuda.ExternalStream(L.lib.nk_stream(ctx)))
    a_h = _rand(rows * k, 0, 3, -2.0, 2.0, start=rank * rows * k)   # this rank's rows of the seed-3 stream
    b_h = _rand(m * k, 0, 4, -2.0, 2.0)
    a, b, a1 = _alloc(ctx, rows * k), _alloc(ctx, m * k), _alloc(ctx, rows * k)
    _upload(ctx, a, a_h); _upload(ctx, b, b_h)
    t, y, g = _alloc(ctx, N), _alloc(ctx, N), _alloc(ctx, N)
    ga = _alloc(ctx, rows * k)
    gb_t, gb = _torch_view_of(ctx, local_rank, m * k)
    ca, pa = _cfg([rows, 1, k]); cb, pb = _cfg([1, m, k]); co, po = _cfg([rows, m, k])

    def forward():
        L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL, L.NK_F32, 3, t, po, a, pa, b, pb, -1), ctx)
        L.check(L.lib.nk_broadcast(ctx, L.NK_OP_ADD, L.NK_F32, 3, y, po, t, po, b, pb, -1), ctx)
        L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, t, po, y, po, -1), ctx)

    def backward():
        # error of sum(tanh(...)) is all ones: g = tanh'(y); da = sum_j g*b; db = sum_i g*(a+1), then the ranks' partials meet
        L.check(L.lib.nk_unary(ctx, L.FUN["tanh"], L.NK_F32, 3, g, po, y, po, 0), ctx)
        L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, ga, pa, b, pb, g, po, 0), ctx)
        L.check(L.lib.nk_scalar_binary(ctx, L.NK_OP_ADD, L.NK_F32, 3, a1, pa, a, pa, 1.0, -1), ctx)
        L.check(L.lib.nk_broadcast(ctx, L.NK_OP_MUL_BOTH, L.NK_F32, 3, gb, pb, a1, pa, g, po, 0), ctx)
        dist.all_reduce(gb_t, op=dist.ReduceOp.SUM)

    timer = _Timer(dev, dist)
    fwd_ms = timer(forward, 1, 3)
    bwd_ms = timer(backward, 1, 3)
    # spot check on this rank: a window of the forward result and one column set of da against float64 numpy
    win = 2048
    got = _download(ctx, t, win, start=N - win)
    idx = np.arange(N - win, N, dtype=np.int64)
    i, j, kk = idx // (m * k), (idx // k) % m, idx % k
    u = (a_h[i * k + kk] * b_h[j * k + kk]).astype(np.float32) + b_h[j * k + kk]
    ok_fwd = bool(np.abs(got - np.tanh(u.astype(np.float64))).max() <= 2e-7 * 4)
    gb_all = _download(ctx, gb, m * k)
    flags = torch.tensor([1.0 if ok_fwd else 0.0, float(np.isfinite(gb_all).all())], dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    fwd_bytes = world * 4.0 * ((N + rows * k + m * k) + (2 * N + m * k) + 2 * N)
    bwd_bytes = world * 4.0 * (2 * N + (N + rows * k + m * k) * 2)
    out = {"n_gpus": world, "rows_per_gpu": rows, "outputs_total": world * N,
           "forward_ms": fwd_ms, "forward_gbs_total": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
           "backward_ms": bwd_ms, "backward_gbs_total": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
           "frac_of_hbm_peak_forward": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / (world * hbm_peak_gbs),
           "frac_of_hbm_peak_backward": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / (world * hbm_peak_gbs),
           "collective": "one NCCL all-reduce of the 8 MiB partial gradient of b per backward pass",
           "forward_window_matches_numpy": bool(flags[0].item() == 1.0), "gradient_finite": bool(flags[1].item() == 1.0),
           "note": "forward = mul-broadcast, add-broadcast, tanh (op by op, as the reference evaluates it); F32 tanh is FP64-bound"}
    for buf in (a, b, a1, t, y, g, ga, gb):
        L.lib.nk_free(ctx, buf)
    return out


def xconv_sharded(dev, dist, rank, world, local_rank, scale=1):
    """Image gradient and kernel gradient of config 5 under the forward pass's row split. With scale > 1 (smaller
    image) rank 0 also recomputes both gradients alone and compares."""
    import torch
    ctx = dev.ctx
    torch.cuda.set_stream(torch.cuda.ExternalStream(L.lib.nk_stream(ctx)))
    B, Cn, H, W, KH = 8, 32, 2048 // scale, 2048 // scale, 5
    OH, OW = H - KH + 1, W - KH + 1
    halo = KH - 1
    # image-gradient rows [lo, hi) of the H image rows; error rows needed: [lo - halo, hi) clipped to [0, OH)
    gs = plan_image_grad_slabs(H, world, halo)[rank]
    lo, hi, e_lo, e_hi = gs.lo, gs.hi, gs.err_lo, gs.err_hi
    re = gs.err_len                                    # error rows held for the image gradient
    k_h = np.empty(Cn * KH * KH, dtype=np.float32)
    L.lib.nk_jrand_fill(L.NK_F32, 1, 6, 0.0, 0.2, k_h.ctypes.data_as(C.c_void_p), k_h.size)
    err_rows = np.empty((B, re, OW), dtype=np.float32)
    for b in range(B):
        err_rows[b] = _rand(re * OW, 0, 9, -1.0, 1.0, start=b * OH * OW + e_lo * OW).reshape(re, OW)
    d_k, d_e = _alloc(ctx, k_h.size), _alloc(ctx, B * re * OW)
    _upload(ctx, d_k, k_h); _upload(ctx, d_e, err_rows)
    # local drain of the deconvolution: re + halo rows; rows [lo - e_lo, lo - e_lo + (hi - lo)) of it are this rank's
    d_ga = _alloc(ctx, B * Cn * (re + halo) * W)
    c_ga, p_ga = _cfg([B, Cn, re + halo, W]); c_k, p_k = _cfg([1, Cn, KH, KH]); c_e, p_e = _cfg([B, 1, re, OW])

    def grad_image():
        L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_ga, p_ga, d_k, p_k, d_e, p_e, 0), ctx)

    # kernel gradient: this rank's error rows [f_lo, f_hi) of the forward split and image rows [f_lo, f_hi + halo)
    f = plan_slabs(OH, world, halo)[rank]
    rf = f.out_len
    img = np.empty((B * Cn, f.in_len, W), dtype=np.float32)
    for pl in range(B * Cn):
        img[pl] = _rand(f.in_len * W, 0, 5, 0.0, 1.0, start=pl * H * W + f.in_lo * W).reshape(f.in_len, W)
    err_f = np.empty((B, rf, OW), dtype=np.float32)
    for b in range(B):
        err_f[b] = _rand(rf * OW, 0, 9, -1.0, 1.0, start=b * OH * OW + f.out_lo * OW).reshape(rf, OW)
    d_img, d_ef = _alloc(ctx, img.size), _alloc(ctx, err_f.size)
    _upload(ctx, d_img, img); _upload(ctx, d_ef, err_f)
    gk_t, d_gk = _torch_view_of(ctx, local_rank, Cn * KH * KH)
    c_img, p_img = _cfg([B, Cn, f.in_len, W]); c_ef, p_ef = _cfg([B, 1, rf, OW])

    def grad_kernel():
        L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, d_gk, p_k, d_img, p_img, d_ef, p_ef, 0), ctx)
        dist.all_reduce(gk_t, op=dist.ReduceOp.SUM)

    timer = _Timer(dev, dist)
    ga_ms = timer(grad_image, 2, 10)
    ga_kernel = dev.last_kernel()
    gk_ms = timer(grad_kernel, 2, 10)
    gk_kernel = dev.last_kernel()
    flops = 2.0 * B * OH * OW * Cn * KH * KH
    out = {"n_gpus": world, "image": [B, Cn, H, W], "grad_image_ms": ga_ms, "grad_image_tflops_total": flops / (ga_ms * 1e-3) / 1e12,
           "grad_image_kernel": ga_kernel, "grad_kernel_ms": gk_ms, "grad_kernel_tflops_total": flops / (gk_ms * 1e-3) / 1e12,
           "grad_kernel_kernel": gk_kernel,
           "split": "rows of the image gradient / of the error; error halo of 4 rows above; kernel gradient = partials + all-reduce of 800 values"}

    if scale > 1:
        # gather the ranks' rows on rank 0 (host side, small) and compare with a single-GPU computation of the whole thing
        grad_image(); grad_kernel()
        dev.sync()
        mine = _download(ctx, d_ga, B * Cn * (re + halo) * W).reshape(B, Cn, re + halo, W)[:, :, lo - e_lo: lo - e_lo + (hi - lo), :]
        parts = [None] * world
        dist.all_gather_object(parts, mine)
        gk = _download(ctx, d_gk, Cn * KH * KH)
        if rank == 0:
            full_e = np.empty((B, OH, OW), dtype=np.float32)
            for b in range(B):
                full_e[b] = _rand(OH * OW, 0, 9, -1.0, 1.0, start=b * OH * OW).reshape(OH, OW)
            full_a = _rand(B * Cn * H * W, 0, 5, 0.0, 1.0)
            dE, dA, dGA, dGK = _alloc(ctx, full_e.size), _alloc(ctx, full_a.size), _alloc(ctx, B * Cn * H * W), _alloc(ctx, Cn * KH * KH)
            _upload(ctx, dE, full_e); _upload(ctx, dA, full_a)
            cA, pA = _cfg([B, Cn, H, W]); cE, pE = _cfg([B, 1, OH, OW])
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, dGA, pA, d_k, p_k, dE, pE, 0), ctx)
            L.check(L.lib.nk_conv(ctx, L.NK_F32, 4, dGK, p_k, dA, pA, dE, pE, 0), ctx)
            want_a = _download(ctx, dGA, B * Cn * H * W).reshape(B, Cn, H, W)
            want_k = _download(ctx, dGK, Cn * KH * KH)
            got_a = np.concatenate(parts, axis=2)
            out["grad_image_equals_single_gpu"] = bool(np.array_equal(got_a, want_a))
            out["grad_kernel_rel_err_vs_single_gpu"] = float(np.abs(gk - want_k).max() / np.abs(want_k).max())
            for buf in (dE, dA, dGA, dGK):
                L.lib.nk_free(ctx, buf)
        dist.barrier()
    for buf in (d_k, d_e, d_ga, d_img, d_ef, d_gk):
        L.lib.nk_free(ctx, buf)
    return out


def run_sharded_extra(dev, dist, rank, world, local_rank, hbm_peak_gbs):
    out = {}
    for name, fn in (("cfg5_gradients_sharded_check_scale4", lambda: xconv_sharded(dev, dist, rank, world, local_rank, scale=4)),
                     ("cfg5_gradients_sharded", lambda: xconv_sharded(dev, dist, rank, world, local_rank, scale=1)),
                     ("cfg3_sharded_rows", lambda: broadcast_sharded(dev, dist, rank, world, local_rank, hbm_peak_gbs))):
        try:
            out[name] = fn()
        except Exception as e:   # every rank must keep taking part in the later collectives: report and go on
            out[name] = {"error": repr(e)}
            dev.sync()
    return out
