"""Host side of the DLPack exchange, exercised without a device: the exported structure and
the lifetime of the exporting array."""

import ctypes as C
import gc

import numpy as np

from dpnp_b200.tensor import _dlpack as D


class _Queue:
    device = 3


class _FakeArray:
    dtype = np.dtype("f4")
    ndim = 2
    shape = (3, 4)
    strides = (8, 2)
    _ptr = 0x7000
    sycl_queue = _Queue()


def test_exported_tensor_describes_the_array_and_is_released():
    x = _FakeArray()
    cap = D.to_dlpack_capsule(x)
    assert D._api.PyCapsule_IsValid(cap, b"dltensor")
    m = C.cast(D._api.PyCapsule_GetPointer(cap, b"dltensor"), C.POINTER(D.DLManagedTensor)).contents
    t = m.dl_tensor
    assert t.data == 0x7000 and t.ndim == 2 and t.byte_offset == 0
    assert (t.device.device_type, t.device.device_id) == (D.kDLCUDA, 3)
    assert (t.dtype.code, t.dtype.bits, t.dtype.lanes) == (2, 32, 1)
    assert [t.shape[i] for i in range(2)] == [3, 4] and [t.strides[i] for i in range(2)] == [8, 2]
    n = len(D._exported)
    m.deleter(C.pointer(m))                       # what a consumer does when it is done
    assert len(D._exported) == n - 1
    # a capsule nobody consumed releases the array when it is collected
    cap2 = D.to_dlpack_capsule(x)
    n = len(D._exported)
    del cap2
    gc.collect()
    assert len(D._exported) == n - 1
    assert D.dlpack_device(x) == (D.kDLCUDA, 3)
