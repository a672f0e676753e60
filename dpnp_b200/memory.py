"""Execution queues and device memory.

``StreamQueue`` stands where the reference carries a ``dpctl.SyclQueue``: it
names a CUDA device and one in-order ``cudaStream_t`` on it.  Work submitted to
one queue runs in submission order, which is the guarantee the reference
obtains from ``SequentialOrderManager`` (dpnp/tensor/_elementwise_common.py:240-254).

``MemoryUSMDevice`` owns one block of the stream-ordered pool and replaces
``dpctl.memory.MemoryUSMDevice`` as wrapped by dpnp/memory/_memory.py:36-110.
Freeing is ordered after the work already queued on the owning stream, so a
block may be released while kernels that use it are still in flight.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

from . import _lib
from ._lib import check, lib
from ._lib import native as _native

__all__ = [
    "StreamQueue", "get_default_queue", "MemoryUSMDevice", "MemoryUSMShared", "MemoryUSMHost",
    "create_data", "PinnedHostBuffer", "copy_host_to_device", "copy_device_to_host", "pool_stats", "pool_trim", "pool_set_limit", "ExecutionPlacementError",
]


class ExecutionPlacementError(Exception):
    """Arrays of one operation live on different devices/queues
    (mirrors dpctl.utils.ExecutionPlacementError)."""


class StreamQueue:
    """A CUDA device ordinal plus one in-order stream on that device."""

    __slots__ = ("device", "_stream", "__weakref__")

    def __init__(self, device: int = 0, stream: int | None = None):
        self.device = int(device)
        if stream is None:
            check(lib.dpb_set_device(self.device))
            h = C.c_void_p()
            check(lib.dpb_stream_create(C.byref(h)))
            self._stream = h.value or 0
        else:
            self._stream = int(stream)

    @property
    def stream(self) -> int:
        """The cudaStream_t as an integer."""
        return self._stream

    # names used by code written against dpctl
    @property
    def sycl_device(self):
        return self.device

    def activate(self) -> None:
        check(lib.dpb_set_device(self.device))

    def wait(self) -> None:
        self.activate()
        check(lib.dpb_stream_synchronize(C.c_void_p(self._stream)))

    synchronize = wait

    def __eq__(self, other):
        return (
            isinstance(other, StreamQueue)
            and other.device == self.device
            and other._stream == self._stream
        )

    def __hash__(self):
        return hash((self.device, self._stream))

    def __repr__(self):
        return f"<StreamQueue cuda:{self.device} stream=0x{self._stream:x}>"


_default_queues: dict[int, StreamQueue] = {}
_default_lock = threading.Lock()
_current_device = [None]


def _require_device() -> None:
    if _lib.device_count() == 0:
        raise RuntimeError(
            "dpnp_b200 needs a CUDA device: none is visible and there is no CPU fallback"
        )


def get_default_queue(device: int | None = None) -> StreamQueue:
    """The library-wide queue of `device` (default: the selected device)."""
    if device is None:
        if _current_device[0] is None:
            # DPNP_B200_DEVICE: ordinal of the device new arrays go to when none is named (the
            # reference reads its default device from the environment too, dpnp/config.py:32-59)
            _current_device[0] = int(os.environ.get("DPNP_B200_DEVICE", "0"))
        device = _current_device[0]
    q = _default_queues.get(device)
    if q is None:
        with _default_lock:
            q = _default_queues.get(device)
            if q is None:
                _require_device()
                q = StreamQueue(device)
                _default_queues[device] = q
    return q


def select_default_device(device: int) -> None:
    """Choose the device new arrays are allocated on when none is given."""
    _current_device[0] = int(device)


def normalize_queue(sycl_queue=None, device=None) -> StreamQueue:
    """Queue from the `sycl_queue=` / `device=` keywords accepted by creation functions."""
    if sycl_queue is not None:
        if not isinstance(sycl_queue, StreamQueue):
            raise TypeError(f"expected a StreamQueue, got {type(sycl_queue)}")
        return sycl_queue
    if device is None:
        return get_default_queue()
    if isinstance(device, StreamQueue):
        return device
    if isinstance(device, str):
        # accept "cuda", "cuda:1", "gpu", "gpu:1"
        name, _, idx = device.partition(":")
        if name not in ("cuda", "gpu"):
            raise ValueError(f"unknown device string {device!r}")
        return get_default_queue(int(idx) if idx else 0)
    return get_default_queue(int(device))


class MemoryUSMDevice:
    """A block of device memory from the stream-ordered pool."""

    usm_type = "device"

    def __init__(self, nbytes: int, queue: StreamQueue | None = None):
        nbytes = int(nbytes)
        if nbytes < 0:
            raise ValueError("nbytes must be non-negative")
        self.sycl_queue = queue if queue is not None else get_default_queue()
        self.nbytes = nbytes
        self._ptr = 0
        self._blk = None
        if _native is not None:
            # the block object returns the memory to the pool when its last reference goes
            self._blk = _native.Block(nbytes, self.sycl_queue.device, self.sycl_queue._stream)
            self._ptr = self._blk.ptr
            return
        self.sycl_queue.activate()
        p = C.c_void_p()
        check(lib.dpb_malloc(nbytes, C.c_void_p(self.sycl_queue.stream), C.byref(p)))
        self._ptr = p.value or 0

    @property
    def ptr(self) -> int:
        """Device address of the first byte (dpnp/memory/_memory.py:36-67 adds the same)."""
        return self._ptr

    @property
    def size(self) -> int:
        return self.nbytes

    def __len__(self):
        return self.nbytes

    def free(self) -> None:
        ptr, self._ptr = self._ptr, 0
        blk = getattr(self, "_blk", None)
        if blk is not None:
            self._blk = None
            blk.release()
            return
        if ptr:
            try:
                lib.dpb_set_device(self.sycl_queue.device)
                lib.dpb_free(C.c_void_p(ptr), C.c_void_p(self.sycl_queue.stream))
            except Exception:  # interpreter shutdown
                pass

    if _native is None:
        # (with the shim, the block object inside gives the memory back by itself)
        def __del__(self):
            self.free()

    def __repr__(self):
        return f"<{type(self).__name__} {self.nbytes} bytes at 0x{self._ptr:x} on cuda:{self.sycl_queue.device}>"


class MemoryUSMShared(MemoryUSMDevice):
    """Accepted for API compatibility; backed by device memory."""

    usm_type = "shared"


class MemoryUSMHost(MemoryUSMDevice):
    """Accepted for API compatibility; backed by device memory."""

    usm_type = "host"


class PinnedHostBuffer:
    """Page-locked host memory (cudaHostAlloc) viewed as a NumPy array: the staging
    area for fast host<->device copies."""

    def __init__(self, shape, dtype):
        import numpy as np

        self.dtype = np.dtype(dtype)
        self.shape = (int(shape),) if isinstance(shape, int) else tuple(int(s) for s in shape)
        n = 1
        for s in self.shape:
            n *= s
        self.nbytes = n * self.dtype.itemsize
        p = C.c_void_p()
        check(lib.dpb_host_alloc(self.nbytes, C.byref(p)))
        self._ptr = p.value
        buf = (C.c_char * max(self.nbytes, 1)).from_address(self._ptr)
        self.array = np.frombuffer(buf, dtype=self.dtype, count=n).reshape(self.shape)

    def free(self):
        ptr, self._ptr = self._ptr, 0
        if ptr:
            self.array = None
            try:
                lib.dpb_host_free(C.c_void_p(ptr))
            except Exception:
                pass

    def __del__(self):
        self.free()


def _order_after(owner_queue, other_queue):
    """Make the work queued later on `owner_queue` (in particular the release of a block it owns)
    wait for what has just been queued on `other_queue`."""
    if other_queue is owner_queue or (other_queue.device == owner_queue.device
                                      and other_queue.stream == owner_queue.stream):
        return
    other_queue.activate()
    ev = C.c_void_p()
    check(lib.dpb_event_create(C.byref(ev)))
    try:
        check(lib.dpb_event_record(ev, C.c_void_p(other_queue.stream)))
        check(lib.dpb_stream_wait_event(C.c_void_p(owner_queue.stream), ev))
    finally:
        lib.dpb_event_destroy(ev)


def copy_host_to_device(dst, host_array, queue=None):
    """Enqueue dst[...] = host_array (same dtype, both C-contiguous) without synchronising;
    the host buffer must stay alive until the queue has been waited on.  With a `queue` other
    than the array's own, the array's queue is made to wait for the copy, so that the memory
    cannot return to the pool (freeing is ordered on the owning queue) while the copy runs."""
    u = dst.get_array() if hasattr(dst, "get_array") else dst
    q = queue or u.sycl_queue
    if not (u.flags.c_contiguous and host_array.flags.c_contiguous and u.dtype == host_array.dtype
            and u.size == host_array.size):
        raise ValueError("copy_host_to_device needs matching C-contiguous buffers")
    q.activate()
    check(lib.dpb_memcpy(C.c_void_p(u._ptr), C.c_void_p(host_array.ctypes.data), host_array.nbytes, 0,
                         C.c_void_p(q.stream)))
    _order_after(u.sycl_queue, q)


def copy_device_to_host(host_array, src, queue=None):
    """Enqueue host_array[...] = src without synchronising."""
    u = src.get_array() if hasattr(src, "get_array") else src
    q = queue or u.sycl_queue
    if not (u.flags.c_contiguous and host_array.flags.c_contiguous and u.dtype == host_array.dtype
            and u.size == host_array.size):
        raise ValueError("copy_device_to_host needs matching C-contiguous buffers")
    q.activate()
    check(lib.dpb_memcpy(C.c_void_p(host_array.ctypes.data), C.c_void_p(u._ptr), host_array.nbytes, 1,
                         C.c_void_p(q.stream)))
    _order_after(u.sycl_queue, q)


def create_data(x):
    """Return the memory object behind an array (dpnp/memory/_memory.py:70-110)."""
    base = getattr(x, "usm_data", None)
    if base is None:
        raise TypeError(f"expected an array with device memory, got {type(x)}")
    return base


def pool_stats() -> dict:
    """Counters of the current device's pool."""
    vals = [C.c_size_t() for _ in range(4)]
    check(lib.dpb_pool_stats(*[C.byref(v) for v in vals]))
    keys = ("reserved", "used", "reserved_high", "used_high")
    return {k: v.value for k, v in zip(keys, vals)}


def pool_trim(keep_bytes: int = 0) -> None:
    check(lib.dpb_pool_trim(int(keep_bytes)))


def pool_set_limit(max_live_bytes: int) -> None:
    check(lib.dpb_pool_set_limit(int(max_live_bytes)))
