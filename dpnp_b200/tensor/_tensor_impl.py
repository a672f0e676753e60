"""Python face of the native ``_tensor_impl`` module of the reference
(dpnp/tensor/libtensor/source/tensor_ctors.cpp): same function names and
argument order, implemented by the C ABI of libdpnp_b200.

Every function takes ``sycl_queue`` (a :class:`StreamQueue`) and ``depends``;
work is enqueued on the queue's stream, whose in-order semantics subsume the
event dependencies, and a pair of :class:`Event` placeholders is returned where
the reference returns ``(host_task_event, compute_event)``.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib
from .._lib import check, lib


class Event:
    """Stands for a completed-or-pending operation on an in-order stream."""

    __slots__ = ("_queue",)

    def __init__(self, queue=None):
        self._queue = queue

    def wait(self):
        if self._queue is not None:
            self._queue.wait()


def _events(q):
    e = Event(q)
    return e, e


def _stream(q):
    q.activate()
    return C.c_void_p(q.stream)


def _check_queue(q, *arrays):
    for a in arrays:
        if a.sycl_queue.device != q.device:
            raise ValueError("Execution queue is not compatible with allocation queues")


_nat = _lib.native


def _where(condition, x1, x2, dst, sycl_queue, depends=()):
    _check_queue(sycl_queue, condition, x1, x2, dst)
    if _nat is not None:
        _nat.where(condition._core(), x1._core(), x2._core(), dst._core(), sycl_queue._stream)
        return _events(sycl_queue)
    dc, kc = condition._descriptor()
    d1, k1 = x1._descriptor()
    d2, k2 = x2._descriptor()
    dd, kd = dst._descriptor()
    check(lib.dpb_where(C.byref(dc), C.byref(d1), C.byref(d2), C.byref(dd), _stream(sycl_queue)))
    return _events(sycl_queue)


def _copy_usm_ndarray_into_usm_ndarray(src, dst, sycl_queue, depends=()):
    _check_queue(sycl_queue, src, dst)
    if _nat is not None:
        _nat.copy(src._core(), dst._core(), sycl_queue._stream)
        return _events(sycl_queue)
    ds, ks = src._descriptor()
    dd, kd = dst._descriptor()
    check(lib.dpb_copy_array_into_array(C.byref(ds), C.byref(dd), _stream(sycl_queue)))
    return _events(sycl_queue)


def _full_usm_ndarray(fill_value, dst, sycl_queue, depends=()):
    dd, kd = dst._descriptor()
    bits = np.asarray(fill_value).astype(dst.dtype, casting="unsafe").tobytes()
    buf = C.create_string_buffer(bits, 16)
    check(lib.dpb_full_array(C.byref(dd), buf, _stream(sycl_queue)))
    return _events(sycl_queue)


def _zeros_usm_ndarray(dst, sycl_queue, depends=()):
    if dst.flags.forc:
        sycl_queue.activate()
        check(lib.dpb_memset(C.c_void_p(dst._ptr), 0, dst.nbytes, C.c_void_p(sycl_queue.stream)))
        return _events(sycl_queue)
    return _full_usm_ndarray(0, dst, sycl_queue, depends)


def _array_overlap(a, b) -> bool:
    """True if the byte ranges spanned by the two arrays intersect (the interval test of
    include/utils/memory_overlap.hpp:52-107; dpb_array_overlap is the native form)."""
    ea, eb = a._byte_extent(), b._byte_extent()
    if ea is None or eb is None:
        return False
    return ea[0] < eb[1] and eb[0] < ea[1]


def _same_logical_tensors(a, b) -> bool:
    """Same pointer, type, shape and strides (memory_overlap.hpp:109-151)."""
    return (a._ptr == b._ptr and a.dtype == b.dtype and a.shape == b.shape and a.strides == b.strides)


def _contract_iter(shape, strides):
    """Collapsed (shape, strides, offset) of one array (strided_iters.hpp contract_iter)."""
    nd = len(shape)
    sh = (C.c_int64 * max(nd, 1))(*shape)
    st = (C.c_int64 * max(nd, 1))(*strides)
    off = (C.c_int64 * 4)()
    out = C.c_int()
    check(lib.dpb_simplify_iteration_space(1, nd, sh, st, off, C.byref(out)))
    m = out.value
    return list(sh[:m]), list(st[:m]), off[0]


def _contract_iter_n(shape, *strides_list):
    """Collapse the iteration space shared by several arrays."""
    nd = len(shape)
    k = len(strides_list)
    sh = (C.c_int64 * max(nd, 1))(*shape)
    flat = [s for st in strides_list for s in st]
    st = (C.c_int64 * max(nd * k, 1))(*flat)
    off = (C.c_int64 * 4)()
    out = C.c_int()
    check(lib.dpb_simplify_iteration_space(k, nd, sh, st, off, C.byref(out)))
    m = out.value
    return list(sh[:m]), [list(st[a * m:(a + 1) * m]) for a in range(k)], list(off[:k])


def _contract_iter2(shape, strides1, strides2):
    sh, sts, offs = _contract_iter_n(shape, strides1, strides2)
    return sh, sts[0], offs[0], sts[1], offs[1]


# Default element types of the device (device_support_queries.cpp:50-115): a
# B200 has both fp16 and fp64, so the defaults are those of an fp64-capable device.
def default_device_fp_type(dev=None): return "f8"
def default_device_int_type(dev=None): return "i8"
def default_device_uint_type(dev=None): return "u8"
def default_device_bool_type(dev=None): return "b1"
def default_device_complex_type(dev=None): return "c16"
def default_device_index_type(dev=None): return "i8"
