"""The Device contract a CudaDevice is held to, after src/test/groovy/ut/device/Cross_Device_Type_Spec.groovy
(store/restore :254-313, slices :315-360, counting :362-413, virtual stays virtual :468-505) and
Tensor_Device_Spec.groovy."""
import numpy as np
import pytest

from neureka_b200 import _lib as L
from neureka_b200.backend import CudaBackend
from neureka_b200.device import CudaDevice
from neureka_b200.tensor import Tensor

pytestmark = pytest.mark.gpu


def test_find_by_keyword(device):
    assert CudaBackend.find("cuda") is device
    assert CudaBackend.find("gpu") is device
    assert CudaBackend.find("0") is device and CudaBackend.find("cuda:0") is device and CudaBackend.find("gpu:99") is None
    assert CudaBackend.find("banana") is None
    assert device.props.sm_count > 0 and device.props.cc_major >= 10


def test_store_restore_round_trip(device):
    for dt in (np.float32, np.float64, np.int32, np.int64, np.int16, np.int8):
        t = Tensor.of(dt, [3, 4], np.arange(12))
        before = device.number_of_stored()
        t.to(device)
        assert device.has(t) and t.is_outsourced and device.number_of_stored() == before + 1
        assert t.items.tolist() == list(range(12))
        device.restore(t)
        assert not device.has(t) and not t.is_outsourced
        assert t.items.tolist() == list(range(12))
        assert device.number_of_stored() == before


def test_access_api(device):
    t = Tensor.of(np.float64, [2, 3], [1, 2, 3, 4, 5, 6]).to(device)
    acc = device.access(t)
    assert acc.get_data_size() == 6
    assert acc.read_at(4) == 5
    assert acc.read_array(1, 3).tolist() == [2, 3, 4]
    acc.write(9.5).at(0)
    acc.write(-1).into_range(2, 4)
    assert acc.read_all().tolist() == [9.5, 2, -1, -1, 5, 6]
    acc.write_from(np.array([10, 20, 30, 40.0]), 1).into_range(3, 6)
    assert acc.read_all().tolist() == [9.5, 2, -1, 20, 30, 40]
    acc.write(0).fully()
    assert acc.read_all().tolist() == [0] * 6
    with pytest.raises(ValueError):
        acc.read_array(4, 5)
    with pytest.raises(ValueError):
        device.access(None)
    device.free(t)
    assert not device.has(t)


def test_slices_share_the_parents_data(device):
    a = Tensor.of(np.float32, [4, 6], np.arange(1, 25)).to(device)
    n_data = device.number_of_data_objects()
    b = a[1:4, 0:4]
    assert device.has(b) and device.number_of_data_objects() == n_data
    assert b.ndconf.as_inline_array().tolist() == [3, 4, 6, 1, 4, 1, 1, 0, 1, 1]
    assert b.items.tolist() == [7, 8, 9, 10, 13, 14, 15, 16, 19, 20, 21, 22]
    c = a[0:4:2, 1:5:2]
    assert c.items.tolist() == [2, 4, 14, 16]
    # a slice made on the host moves with its root
    h = Tensor.of(np.float64, [3, 3], np.arange(9))
    s = h[1:3, 1:3]
    s.to(device)
    assert device.has(h) and device.has(s)
    assert s.items.tolist() == [4, 5, 7, 8]
    device.restore(h)
    assert not device.has(s) and s.items.tolist() == [4, 5, 7, 8]
    device.restore(a)


def test_virtual_tensors_stay_virtual(device):
    t = Tensor.of(np.float32, [100, 100], 4.0)
    assert t.is_virtual
    t.to(device)
    assert t.is_virtual and device.access(t).get_data_size() == 1
    assert t.items[:3].tolist() == [4, 4, 4] and t.items.size == 10_000
    t.set_is_virtual(False)
    assert device.access(t).get_data_size() == 10_000
    assert np.all(device.access(t).read_all() == 4.0)
    device.restore(t)
    assert t.items.size == 10_000


def test_gradient_moves_with_its_tensor(device):
    t = Tensor.of(np.float32, [2], [1, 2]).set_rqs_gradient(True)
    t.gradient = Tensor.of(np.float32, [2], [5, 6])
    t.to(device)
    assert device.has(t.gradient)
    device.restore(t)
    assert not t.gradient.is_outsourced and t.gradient.items.tolist() == [5, 6]


def test_out_of_memory_is_reported(device):
    buf = __import__("ctypes").c_void_p()
    st = L.lib.nk_alloc(device.ctx, L.NK_F64, 1 << 45, __import__("ctypes").byref(buf))
    assert st == L.NK_ERR_OOM
    assert b"memory" in L.lib.nk_last_error(device.ctx).lower()
    # the context is still usable
    t = Tensor.of(np.float32, [2], [1, 2]).to(device)
    assert t.items.tolist() == [1, 2]
    device.restore(t)


def test_sizes_that_would_wrap_are_refused_before_any_allocation(device):
    """n_elems * element size must not wrap (a wrapped allocation would succeed and claim memory it does not have), and a
    view's element count is checked before each multiplication (eight extents of 2^16 wrap int64 to 0)."""
    import ctypes as C
    buf = C.c_void_p()
    assert L.lib.nk_alloc(device.ctx, L.NK_F64, 1 << 61, C.byref(buf)) == L.NK_ERR_OOM and not buf
    assert L.lib.nk_alloc(device.ctx, L.NK_F64, 1 << 43, C.byref(buf)) == L.NK_ERR_OOM and not buf     # 64 TiB: the driver refuses
    assert L.lib.nk_wrap(device.ctx, L.NK_F32, C.c_void_p(256), 1 << 61, C.byref(buf)) == L.NK_ERR_BAD_ARG
    L.check(L.lib.nk_alloc(device.ctx, L.NK_F32, 16, C.byref(buf)), device.ctx)
    try:
        rank = 8
        cfg = np.array([1 << 16] * rank + [0] * rank + [1] * rank + [0] * rank + [1] * rank, dtype=np.int32)   # stride-0 view, 2^128 elements
        st = L.lib.nk_unary(device.ctx, L.FUN["relu"], L.NK_F32, rank, buf, cfg.ctypes.data_as(C.POINTER(C.c_int32)),
                            buf, cfg.ctypes.data_as(C.POINTER(C.c_int32)), -1)
        assert st == L.NK_ERR_UNSUPPORTED
        assert b"too large" in L.lib.nk_last_error(device.ctx)
    finally:
        L.lib.nk_free(device.ctx, buf)


def test_pooled_allocations_are_reused_and_shared_ones_export(device):
    """nk_alloc / nk_free go through the stream-ordered pool: a freed block comes back for the next request of the same
    size without a device-wide wait; pooled memory has no IPC handle, nk_alloc_shared memory has."""
    import ctypes as C
    ctx = device.ctx
    n = 1 << 22
    seen = set()
    for _ in range(6):
        b = C.c_void_p()
        L.check(L.lib.nk_alloc(ctx, L.NK_F32, n, C.byref(b)), ctx)
        L.check(L.lib.nk_fill(ctx, b, C.c_double(1.0), 0, n), ctx)
        p = C.c_void_p()
        L.lib.nk_buf_info(b, C.byref(p), None, None)
        seen.add(p.value)
        L.check(L.lib.nk_free(ctx, b), ctx)
    assert len(seen) <= 2, "freed blocks were not handed out again"
    handle = (C.c_uint8 * L.NK_IPC_HANDLE_BYTES)()
    b = C.c_void_p()
    L.check(L.lib.nk_alloc(ctx, L.NK_F32, n, C.byref(b)), ctx)
    assert L.lib.nk_ipc_export(ctx, b, handle) == L.NK_ERR_BAD_ARG
    L.check(L.lib.nk_free(ctx, b), ctx)
    L.check(L.lib.nk_alloc_shared(ctx, L.NK_F32, n, C.byref(b)), ctx)
    L.check(L.lib.nk_ipc_export(ctx, b, handle), ctx)
    assert any(handle)
    L.check(L.lib.nk_free(ctx, b), ctx)


def test_null_arguments_of_a_call_are_refused(device):
    """Cross_Device_Type_Spec.groovy:221-252: an ExecutionCall with a null tensor argument is an IllegalArgumentException
    with this very message (AbstractDeviceAlgorithm.java:119-124)."""
    from neureka_b200 import backend as Bk
    from neureka_b200.functions import _execute_on_common_device
    t = Tensor.of(np.float32, [2], [1, 2]).to(device)
    call = Bk.ExecutionCall([t, None], "+", device, -1)
    with pytest.raises(ValueError) as e:
        _execute_on_common_device(call, Bk.backend().implementation_for("+", Bk.BI_ELEMENTWISE))
    assert "Device arguments may not be null!" in str(e.value)
    assert "One or more tensor arguments within the given ExecutionCall instance is null." in str(e.value)
    device.restore(t)


def test_device_counts_tensors_and_data_objects(device):
    """Cross_Device_Type_Spec.groovy:362-413: a stored tensor is one tensor and one data object; a result of an
    operation on it is another of each; a reshaped view is a new tensor on the same data object; dropping them all
    brings both counts back."""
    import gc
    gc.collect()
    initial, initial_data = device.number_of_stored(), device.number_of_data_objects()
    t = Tensor.of(np.float64, [2, 2], [42, 73, 11, 7])
    assert device.number_of_stored() == initial
    t.to(device)
    assert device.number_of_stored() == initial + 1 and device.number_of_data_objects() == initial_data + 1
    t2 = t * 2
    assert t2.items.tolist() == [84, 146, 22, 14]
    assert device.number_of_stored() == initial + 2 and device.number_of_data_objects() == initial_data + 2
    t3 = t.permute(1, 0)
    assert device.has(t3)
    assert device.number_of_stored() == initial + 3 and device.number_of_data_objects() == initial_data + 2
    for x in (t3, t2, t):
        device.free(x)
    del t, t2, t3
    gc.collect()
    assert device.number_of_stored() == initial and device.number_of_data_objects() == initial_data


def test_a_slice_lives_where_its_parent_lives(device):
    """Cross_Device_Type_Spec.groovy:415-466 (AbstractDevice.java:92-99): a slice has no device data of its own. Storing
    the parent outsources the slice with it and adds one data object, not two; here storing the slice first moves its
    root along (the reference throws "Data parent is not outsourced!" at that point -- in a spec it keeps ignored)."""
    a = Tensor.of(np.float32, [2, 3], [1, 2, 3, 4, 5, 6])
    b = a[1:2, 0:3]
    n_data = device.number_of_data_objects()
    assert not device.has(a) and not device.has(b)
    a.to(device)
    assert a.is_outsourced and b.is_outsourced and device.has(a) and device.has(b)
    assert device.number_of_data_objects() == n_data + 1
    assert b.items.tolist() == [4, 5, 6]
    device.restore(a)
    assert not device.has(b) and not b.is_outsourced and b.items.tolist() == [4, 5, 6]
    c = Tensor.of(np.float32, [2, 3], [1, 2, 3, 4, 5, 6])
    d = c[0:1, 1:3]
    d.to(device)
    assert device.has(c) and device.has(d) and device.number_of_data_objects() == n_data + 1
    device.restore(c)


def test_events_order_two_contexts_on_one_device(device):
    """A second context on the same device is a second stream; an event recorded on the first makes the second wait.
    The producer stream fills and squares a buffer many times over (long enough to still be running when the copy is
    queued); the copy on the other stream, ordered by the event, must see the final values."""
    import ctypes as C
    import numpy as np
    from neureka_b200 import _lib as L
    from neureka_b200.ndconf import NDConfiguration as ND

    ctx_a = device.ctx
    ctx_b = C.c_void_p()
    L.check(L.lib.nk_device_open(getattr(device, "ordinal", 0), C.byref(ctx_b)))
    try:
        n = 1 << 24
        src, dst = C.c_void_p(), C.c_void_p()
        L.check(L.lib.nk_alloc(ctx_a, L.NK_F32, n, C.byref(src)), ctx_a)
        L.check(L.lib.nk_alloc(ctx_a, L.NK_F32, n, C.byref(dst)), ctx_a)
        L.check(L.lib.nk_fill(ctx_a, dst, C.c_double(-1.0), 0, n), ctx_a)
        L.check(L.lib.nk_sync(ctx_a), ctx_a)
        ev = C.c_void_p()
        L.check(L.lib.nk_event_create(ctx_a, C.byref(ev)), ctx_a)
        L.check(L.lib.nk_stream_wait_event(ctx_b, ev), ctx_b)          # never recorded: must not block
        cfg = ND.of_shape([n]).as_inline_array()
        pc = cfg.ctypes.data_as(C.POINTER(C.c_int32))
        L.check(L.lib.nk_fill(ctx_a, src, C.c_double(1.0), 0, n), ctx_a)
        for _ in range(40):                                            # src = src + src, 40 times: 2^40
            L.check(L.lib.nk_binary(ctx_a, L.NK_OP_ADD, L.NK_F32, 1, src, pc, src, pc, src, pc, -1), ctx_a)
        L.check(L.lib.nk_event_record(ctx_a, ev), ctx_a)
        L.check(L.lib.nk_stream_wait_event(ctx_b, ev), ctx_b)
        L.check(L.lib.nk_copy(ctx_b, dst, 0, src, 0, n), ctx_b)
        L.check(L.lib.nk_sync(ctx_b), ctx_b)
        got = np.empty(n, dtype=np.float32)
        L.check(L.lib.nk_read(ctx_b, dst, got.ctypes.data_as(C.c_void_p), 0, n), ctx_b)
        assert np.all(got == np.float32(2.0 ** 40))
        assert L.lib.nk_event_free(ev) == L.NK_OK
        assert L.lib.nk_event_record(ctx_a, None) == L.NK_ERR_BAD_ARG
        L.lib.nk_free(ctx_a, src)
        L.lib.nk_free(ctx_a, dst)
    finally:
        L.lib.nk_device_close(ctx_b)


def test_bounded_wait_runs_out_and_is_reported(device):
    """The pipelined kernels wait on mbarriers with a time limit. Here the same wait runs on a barrier nothing ever
    completes, with a 20 ms limit: the kernel returns by itself, the next synchronising call reports NK_ERR_TIMEOUT
    and the context stays usable."""
    import ctypes as C
    import numpy as np
    from neureka_b200 import _lib as L

    waited = C.c_uint64(0)
    assert L.lib.nk_probe_wait_timeout(device.ctx, 20_000_000, C.byref(waited)) == L.NK_OK
    assert 20_000_000 <= waited.value < 500_000_000, waited.value
    assert L.lib.nk_sync(device.ctx) == L.NK_ERR_TIMEOUT
    assert b"gave up waiting" in L.lib.nk_last_error(device.ctx)
    assert L.lib.nk_sync(device.ctx) == L.NK_OK                      # reported once, then clear
    buf = C.c_void_p()
    L.check(L.lib.nk_alloc(device.ctx, L.NK_F32, 16, C.byref(buf)), device.ctx)
    L.check(L.lib.nk_fill(device.ctx, buf, C.c_double(3.0), 0, 16), device.ctx)
    out = np.empty(16, dtype=np.float32)
    L.check(L.lib.nk_read(device.ctx, buf, out.ctypes.data_as(C.c_void_p), 0, 16), device.ctx)
    assert np.all(out == 3.0)
    L.lib.nk_free(device.ctx, buf)
    assert L.lib.nk_probe_wait_timeout(device.ctx, 0, None) == L.NK_ERR_BAD_ARG
