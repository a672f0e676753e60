"""DLPack exchange: ``from_dlpack`` and ``usm_ndarray.__dlpack__`` / ``__dlpack_device__``.

The reference implements the protocol in Cython (dpnp/tensor/_dlpack.pyx: ``to_dlpack_capsule``
:250-380, ``from_dlpack_capsule`` :560-760, ``from_dlpack`` :900-1100) over SYCL USM pointers;
here the ``DLManagedTensor`` is built and read with ctypes over CUDA device pointers
(device type kDLCUDA = 2), so arrays move to and from any CUDA-aware DLPack consumer without
a copy and without passing through the host.
"""

from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib

kDLCPU, kDLCUDA, kDLCUDAHost, kDLCUDAManaged = 1, 2, 3, 13
_CODES = {"i": 0, "u": 1, "f": 2, "c": 5, "b": 6}     # DLDataTypeCode: int, uint, float, complex, bool


class DLDevice(C.Structure):
    _fields_ = [("device_type", C.c_int32), ("device_id", C.c_int32)]


class DLDataType(C.Structure):
    _fields_ = [("code", C.c_uint8), ("bits", C.c_uint8), ("lanes", C.c_uint16)]


class DLTensor(C.Structure):
    _fields_ = [("data", C.c_void_p), ("device", DLDevice), ("ndim", C.c_int32), ("dtype", DLDataType),
                ("shape", C.POINTER(C.c_int64)), ("strides", C.POINTER(C.c_int64)), ("byte_offset", C.c_uint64)]


class DLManagedTensor(C.Structure):
    pass


_DELETER = C.CFUNCTYPE(None, C.POINTER(DLManagedTensor))
DLManagedTensor._fields_ = [("dl_tensor", DLTensor), ("manager_ctx", C.c_void_p), ("deleter", _DELETER)]

_api = C.pythonapi
_api.PyCapsule_New.restype = C.py_object
_api.PyCapsule_New.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p]
_api.PyCapsule_IsValid.restype = C.c_int
_api.PyCapsule_IsValid.argtypes = [C.py_object, C.c_char_p]
_api.PyCapsule_GetPointer.restype = C.c_void_p
_api.PyCapsule_GetPointer.argtypes = [C.py_object, C.c_char_p]
_api.PyCapsule_SetName.restype = C.c_int
_api.PyCapsule_SetName.argtypes = [C.py_object, C.c_char_p]

_NAME, _USED = b"dltensor", b"used_dltensor"
_exported = {}          # address of a live DLManagedTensor -> (struct, shape, strides, array): kept alive


@_DELETER
def _deleter(ptr):
    _exported.pop(C.addressof(ptr.contents), None)


_CAPSULE_DESTRUCTOR = C.CFUNCTYPE(None, C.c_void_p)


@_CAPSULE_DESTRUCTOR
def _capsule_destructor(capsule_addr):
    """A capsule that was never consumed still owns its tensor: release it."""
    try:
        capsule = C.cast(capsule_addr, C.py_object)
        if _api.PyCapsule_IsValid(capsule, _NAME):
            _exported.pop(_api.PyCapsule_GetPointer(capsule, _NAME), None)
    except Exception:                                    # interpreter shutdown: nothing to release
        pass


def to_dlpack_capsule(x):
    """Capsule named "dltensor" that shares the memory of `x`; the array stays alive until the
    consumer calls the deleter."""
    dt = x.dtype
    if dt.kind not in _CODES:
        raise BufferError(f"arrays of type {dt} cannot be exported through DLPack")
    nd = x.ndim
    shape = (C.c_int64 * max(nd, 1))(*x.shape)
    strides = (C.c_int64 * max(nd, 1))(*x.strides)
    m = DLManagedTensor()
    m.dl_tensor.data = x._ptr
    m.dl_tensor.device = DLDevice(kDLCUDA, x.sycl_queue.device)
    m.dl_tensor.ndim = nd
    m.dl_tensor.dtype = DLDataType(_CODES[dt.kind], dt.itemsize * 8, 1)
    m.dl_tensor.shape = shape
    m.dl_tensor.strides = strides
    m.dl_tensor.byte_offset = 0
    m.manager_ctx = None
    m.deleter = _deleter
    _exported[C.addressof(m)] = (m, shape, strides, x)
    return _api.PyCapsule_New(C.addressof(m), _NAME, C.cast(_capsule_destructor, C.c_void_p))


def dlpack_device(x):
    return (kDLCUDA, x.sycl_queue.device)


class _Imported:
    """Owner of an imported DLManagedTensor: calls the producer's deleter when the last array
    built on the memory goes away."""

    def __init__(self, managed_ptr, nbytes, ptr):
        self._managed = managed_ptr
        self.ptr = ptr
        self.nbytes = nbytes

    def __del__(self):
        m = self._managed
        if m and m.contents.deleter:
            m.contents.deleter(m)
        self._managed = None


def from_dlpack(obj, /, *, device=None, copy=None):
    """Array sharing the memory of `obj` (anything with ``__dlpack__``, or a "dltensor" capsule).
    Only CUDA device memory is accepted: nothing is staged through the host."""
    from ..memory import StreamQueue, get_default_queue
    from ._usmarray import usm_ndarray

    q = device if isinstance(device, StreamQueue) else None
    if hasattr(obj, "__dlpack__"):
        # The producer is handed the stream the array will be used on, so that it orders its
        # pending work before this library's first kernel (the stream is a non-blocking one: it
        # does not wait for the legacy default stream by itself).  A producer that does not
        # take the argument gets a device-wide synchronisation instead.  Capsules passed in
        # directly carry no such handshake: their producer's work is the caller's to order.
        if q is None:
            try:
                q = get_default_queue(int(obj.__dlpack_device__()[1]))
            except Exception:
                q = get_default_queue()
        try:
            capsule = obj.__dlpack__(stream=q.stream)
        except (TypeError, ValueError, AssertionError, RuntimeError, BufferError):
            capsule = obj.__dlpack__()
            q.activate()
            _lib.check(_lib.lib.dpb_device_synchronize())
    else:
        capsule = obj
    if not _api.PyCapsule_IsValid(capsule, _NAME):
        raise TypeError("from_dlpack needs an object with __dlpack__ or an unconsumed 'dltensor' capsule")
    managed = C.cast(_api.PyCapsule_GetPointer(capsule, _NAME), C.POINTER(DLManagedTensor))
    t = managed.contents.dl_tensor
    if t.device.device_type not in (kDLCUDA, kDLCUDAManaged):
        raise BufferError(f"DLPack device type {t.device.device_type} is not CUDA device memory")
    if t.dtype.lanes != 1:
        raise BufferError("vector lanes are not supported")
    kinds = {v: k for k, v in _CODES.items()}
    if t.dtype.code not in kinds:
        raise BufferError(f"DLPack type code {t.dtype.code} is not supported")
    kind = kinds[t.dtype.code]
    try:
        dt = np.dtype("?") if kind == "b" else np.dtype(f"{kind}{t.dtype.bits // 8}")
    except TypeError:
        raise BufferError(f"DLPack type ({t.dtype.code}, {t.dtype.bits} bits) is not supported") from None
    shape = tuple(t.shape[i] for i in range(t.ndim))
    if t.strides:
        strides = tuple(t.strides[i] for i in range(t.ndim))
    else:
        strides, acc = [], 1
        for s in reversed(shape):
            strides.append(acc)
            acc *= s
        strides = tuple(reversed(strides))
    _api.PyCapsule_SetName(capsule, _USED)              # the capsule is consumed
    ptr = (t.data or 0) + t.byte_offset
    lo = sum(min(0, (n - 1) * s) for n, s in zip(shape, strides)) if all(shape) else 0
    hi = sum(max(0, (n - 1) * s) for n, s in zip(shape, strides)) if all(shape) else 0
    owner = _Imported(managed, (hi - lo + 1) * dt.itemsize if all(shape) else 0, ptr + lo * dt.itemsize)
    if q is None or q.device != t.device.device_id:
        q = get_default_queue(t.device.device_id)
    owner.sycl_queue = q
    res = usm_ndarray._view(owner, ptr, shape, strides, dt, q)
    if copy:
        from ._copy_utils import copy as _copy
        return _copy(res)
    return res
