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
    assert CudaBackend.find("0") is device
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
