"""``usm_ndarray``: the strided view over device memory that every kernel sees.

Restates the array object of the reference (fields dpnp/tensor/_usmarray.pxd:81-111,
constructor dpnp/tensor/_usmarray.pyx:327-488, contiguity flags
dpnp/tensor/_stride_utils.pyx:62-229, basic slicing dpnp/tensor/_slicing.pyx:128-...)
on top of a raw CUDA device pointer: ``_ptr`` is the address of element
``[0, ..., 0]``, ``strides`` are in ELEMENTS, ``flags`` uses C=1, F=2, W=4,
``usm_data`` is the owning :class:`~dpnp_b200.memory.MemoryUSMDevice`.
"""

from __future__ import annotations

import ctypes as C
import operator

import numpy as np

from .. import _lib
from .._lib import _TYPENUM, FLAG_C, FLAG_F, FLAG_W, check, dpb_array, lib
from .._lib import native as _native
from ..memory import MemoryUSMDevice, StreamQueue, get_default_queue, normalize_queue


def _dense_strides(shape, order="C"):
    st = [0] * len(shape)
    acc = 1
    rng = range(len(shape) - 1, -1, -1) if order == "C" else range(len(shape))
    for i in rng:
        st[i] = acc
        acc *= shape[i]
    return tuple(st)


def _contig_flags(shape, strides) -> int:
    """C/F contiguity bits of a shape/strides pair."""
    n = 1
    for s in shape:
        n *= s
    if n == 0 or len(shape) == 0:
        return FLAG_C | FLAG_F
    is_c = True
    acc = 1
    for i in range(len(shape) - 1, -1, -1):
        if shape[i] == 1:
            continue
        if strides[i] != acc:
            is_c = False
            break
        acc *= shape[i]
    is_f = True
    acc = 1
    for i in range(len(shape)):
        if shape[i] == 1:
            continue
        if strides[i] != acc:
            is_f = False
            break
        acc *= shape[i]
    return (FLAG_C if is_c else 0) | (FLAG_F if is_f else 0)


class Flags:
    """Read-only view of an array's flags (``x.flags["C"]``, ``x.flags.c_contiguous``...)."""

    __slots__ = ("_v",)

    def __init__(self, v):
        self._v = v

    @property
    def c_contiguous(self):
        return bool(self._v & FLAG_C)

    @property
    def f_contiguous(self):
        return bool(self._v & FLAG_F)

    @property
    def writable(self):
        return bool(self._v & FLAG_W)

    @property
    def fc(self):
        return self.c_contiguous and self.f_contiguous

    @property
    def forc(self):
        return self.c_contiguous or self.f_contiguous

    @property
    def contiguous(self):
        return self.forc

    def __getitem__(self, key):
        key = key.upper() if isinstance(key, str) else key
        if key in ("C", "C_CONTIGUOUS"):
            return self.c_contiguous
        if key in ("F", "F_CONTIGUOUS"):
            return self.f_contiguous
        if key in ("W", "WRITABLE"):
            return self.writable
        if key == "FC":
            return self.fc
        if key == "FORC":
            return self.forc
        raise KeyError(key)

    def __repr__(self):
        return (f"  C_CONTIGUOUS : {self.c_contiguous}\n  F_CONTIGUOUS : {self.f_contiguous}\n"
                f"  WRITABLE : {self.writable}")


def _normalize_shape(shape):
    if isinstance(shape, (int, np.integer)):
        shape = (int(shape),)
    try:
        shape = tuple(operator.index(s) for s in shape)
    except TypeError:
        raise TypeError("Argument shape must be a non-negative integer, or a list/tuple of such integers.") from None
    if any(s < 0 for s in shape):
        raise ValueError("negative dimensions are not allowed")
    return shape


class usm_ndarray:
    """N-dimensional strided array over CUDA device memory."""

    __array_priority__ = 100.0
    # per-object caches, filled on first use (class-level defaults keep construction cheap)
    _desc_cache = None
    _core_cache = None
    _bcast_cache = None
    _extent_cache = 0
    _array_namespace = None
    _usm_type = "device"

    def __init__(self, shape, dtype=None, strides=None, buffer="device", offset=0, order="C",
                 buffer_ctor_kwargs=None, array_namespace=None):
        shape = _normalize_shape(shape)
        if len(shape) > _lib.MAX_ND:
            raise ValueError(f"arrays with more than {_lib.MAX_ND} dimensions are not supported")
        if dtype is None:
            dtype = np.float64
        dtype = np.dtype(dtype)
        _lib.typenum_of(dtype)  # TypeError for unsupported types
        if order not in ("C", "F", "c", "f"):
            raise ValueError("Order can be only 'C' or 'F'")
        order = order.upper()
        if strides is None:
            strides = _dense_strides(shape, order)
        else:
            strides = tuple(operator.index(s) for s in strides)
            if len(strides) != len(shape):
                raise ValueError("strides must have one entry per dimension")
        offset = operator.index(offset)
        nelems = 1
        lo = hi = 0
        for sh, st in zip(shape, strides):
            nelems *= sh
        if nelems > 0:
            for sh, st in zip(shape, strides):
                span = st * (sh - 1)
                if span < 0:
                    lo += span
                else:
                    hi += span
        itemsize = dtype.itemsize
        kwargs = dict(buffer_ctor_kwargs or {})
        if isinstance(buffer, str):
            if buffer not in ("device", "shared", "host"):
                raise ValueError(f"buffer='{buffer}' is not understood; expected 'device', 'shared' or 'host'")
            queue = kwargs.get("queue") or get_default_queue()
            self._usm_type = buffer
            nbytes = (offset + hi + 1) * itemsize if nelems > 0 else itemsize
            if offset + lo < 0:
                raise ValueError("offset and strides address memory before the buffer")
            mem = MemoryUSMDevice(nbytes, queue)
        elif isinstance(buffer, MemoryUSMDevice):
            mem = buffer
            self._usm_type = getattr(buffer, "usm_type", "device")
        elif isinstance(buffer, usm_ndarray):
            mem = buffer.usm_data
            self._usm_type = buffer.usm_type
            offset += (buffer._ptr - mem.ptr) // buffer.dtype.itemsize if buffer.dtype.itemsize == itemsize else 0
            if buffer.dtype.itemsize != itemsize:
                raise ValueError("buffer array must have the same item size")
        else:
            raise ValueError(f"buffer of type {type(buffer)} is not supported")
        if nelems > 0:
            if (offset + lo) * itemsize < 0 or (offset + hi + 1) * itemsize > mem.nbytes:
                raise ValueError("shape, strides and offset address memory outside the buffer")
        self._base = mem
        self._ptr = mem.ptr + offset * itemsize
        self._shape = shape
        self._strides = strides
        self._dtype = dtype
        self._flags = _contig_flags(shape, strides) | FLAG_W
        self._queue = mem.sycl_queue
        if array_namespace is not None:
            self._array_namespace = array_namespace

    # ------------------------------------------------------------ internals
    @classmethod
    def _view(cls, base_mem, ptr, shape, strides, dtype, queue, writable=True, usm_type="device"):
        """Unchecked construction of a view (used by slicing and manipulation)."""
        self = cls.__new__(cls)
        self._base = base_mem
        self._ptr = ptr
        self._shape = tuple(shape)
        self._strides = tuple(strides)
        self._dtype = dtype
        self._flags = _contig_flags(self._shape, self._strides) | (FLAG_W if writable else 0)
        self._queue = queue
        if usm_type != "device":
            self._usm_type = usm_type
        return self

    @classmethod
    def _new_dense(cls, shape, dtype, queue, order_flag=FLAG_C, usm_type="device"):
        """New array of `shape` (a tuple of non-negative ints) in C (FLAG_C) or F (FLAG_F) order
        on `queue`: what ``usm_ndarray(shape, dtype, buffer=usm_type, order=...)`` builds, minus
        the argument checks -- the allocation of every elementwise and reduction result."""
        self = cls.__new__(cls)
        n = 1
        for d in shape:
            n *= d
        self._base = mem = MemoryUSMDevice((n if n > 0 else 1) * dtype.itemsize, queue)
        self._ptr = mem._ptr
        self._shape = shape
        if len(shape) == 1:
            self._strides = (1,)
            self._flags = FLAG_C | FLAG_F | FLAG_W
        else:
            self._strides = _dense_strides(shape, "C" if order_flag == FLAG_C else "F")
            # a dense array is contiguous both ways when at most one extent exceeds 1
            big = 0
            for d in shape:
                if d > 1:
                    big += 1
            self._flags = ((FLAG_C | FLAG_F) if (n == 0 or big <= 1) else order_flag) | FLAG_W
        self._dtype = dtype
        self._queue = queue
        if usm_type != "device":
            self._usm_type = usm_type
        return self

    def _core(self):
        """The array's view for the pybind11 shim (built once per array object)."""
        c = self._core_cache
        if c is None:
            c = self._core_cache = _native.ArrayCore(self._ptr, _TYPENUM[self._dtype], self._flags,
                                                     self._queue.device, self._shape, self._strides)
        return c

    def _like(self, ptr, shape, strides):
        return usm_ndarray._view(self._base, ptr, shape, strides, self._dtype, self._queue,
                                 bool(self._flags & FLAG_W), self._usm_type)

    def _descriptor(self):
        """(dpb_array, keepalive) for the C ABI; built once per array object."""
        cached = self._desc_cache
        if cached is not None:
            return cached
        nd = len(self._shape)
        sh = (C.c_int64 * max(nd, 1))(*self._shape)
        st = (C.c_int64 * max(nd, 1))(*self._strides)
        d = dpb_array()
        d.data = self._ptr
        d.nd = nd
        d.typenum = _lib.typenum_of(self._dtype)
        d.flags = self._flags
        d.device = self._queue.device
        d.shape = C.cast(sh, C.POINTER(C.c_int64))
        d.strides = C.cast(st, C.POINTER(C.c_int64))
        self._desc_cache = (d, (sh, st))
        return self._desc_cache

    def _byte_extent(self):
        """Half-open range of byte addresses the array can touch (None when empty)."""
        ext = self._extent_cache
        if ext != 0:
            return ext
        lo = hi = 0
        empty = False
        for sh, st in zip(self._shape, self._strides):
            if sh == 0:
                empty = True
                break
            span = st * (sh - 1)
            if span < 0:
                lo += span
            else:
                hi += span
        item = self._dtype.itemsize
        ext = None if empty else (self._ptr + lo * item, self._ptr + (hi + 1) * item)
        self._extent_cache = ext
        return ext

    # ----------------------------------------------------------- attributes
    @property
    def shape(self):
        return self._shape

    @shape.setter
    def shape(self, new_shape):
        from ._manipulation_functions import reshape

        r = reshape(self, new_shape, copy=False)
        self._shape, self._strides, self._flags = r._shape, r._strides, r._flags
        self._desc_cache = None
        self._core_cache = None
        self._bcast_cache = None
        self._extent_cache = 0

    @property
    def strides(self):
        """Strides in elements."""
        return self._strides

    @property
    def dtype(self):
        return self._dtype

    @property
    def ndim(self):
        return len(self._shape)

    @property
    def size(self):
        n = 1
        for s in self._shape:
            n *= s
        return n

    @property
    def itemsize(self):
        return self._dtype.itemsize

    @property
    def nbytes(self):
        return self.size * self._dtype.itemsize

    @property
    def flags(self):
        return Flags(self._flags)

    @property
    def usm_data(self):
        return self._base

    base = usm_data

    @property
    def usm_type(self):
        return self._usm_type

    @property
    def sycl_queue(self) -> StreamQueue:
        return self._queue

    @property
    def sycl_device(self):
        return self._queue.device

    @property
    def device(self):
        return self._queue

    @property
    def _pointer(self):
        return self._ptr

    @property
    def _element_offset(self):
        return (self._ptr - self._base.ptr) // self._dtype.itemsize

    @property
    def T(self):
        return self._like(self._ptr, self._shape[::-1], self._strides[::-1])

    @property
    def mT(self):
        if self.ndim < 2:
            raise ValueError("array.mT requires array to have at least 2 dimensions.")
        sh = self._shape[:-2] + (self._shape[-1], self._shape[-2])
        st = self._strides[:-2] + (self._strides[-1], self._strides[-2])
        return self._like(self._ptr, sh, st)

    @property
    def __cuda_array_interface__(self):
        """Zero-copy export (strides in bytes; None when C-contiguous)."""
        item = self._dtype.itemsize
        return {
            "shape": self._shape,
            "typestr": self._dtype.str,
            "data": (self._ptr, not bool(self._flags & FLAG_W)),
            "version": 3,
            "strides": None if (self._flags & FLAG_C) else tuple(s * item for s in self._strides),
            "stream": self._queue.stream or None,
        }

    def __dlpack__(self, *, stream=None, max_version=None, dl_device=None, copy=None):
        """DLPack capsule sharing this array's memory (dpnp/tensor/_usmarray.pyx:1130-1260).  Work
        queued on the array's stream is finished first unless the consumer passes ``stream=-1``."""
        from ._dlpack import to_dlpack_capsule

        if stream != -1:
            self._queue.wait()
        return to_dlpack_capsule(self)

    def __dlpack_device__(self):
        from ._dlpack import dlpack_device

        return dlpack_device(self)

    def __array_namespace__(self, api_version=None):
        from .. import tensor

        return self._array_namespace or tensor

    # ---------------------------------------------------------- conversions
    def __len__(self):
        if self.ndim == 0:
            raise TypeError("len() of unsized object")
        return self._shape[0]

    def _scalar(self):
        if self.size != 1:
            raise ValueError("only size-1 arrays can be converted to Python scalars")
        from ._copy_utils import asnumpy

        return asnumpy(self).reshape(())[()]

    def __bool__(self):
        if self.size == 1:
            return bool(self._scalar())
        if self.size == 0:
            raise ValueError("The truth value of an empty array is ambiguous")
        raise ValueError(
            "The truth value of an array with more than one element is ambiguous. Use dpnp.any() or dpnp.all()")

    def __float__(self):
        return float(self._scalar())

    def __int__(self):
        return int(self._scalar())

    def __complex__(self):
        return complex(self._scalar())

    def __index__(self):
        if self._dtype.kind not in "biu":
            raise IndexError("only integer arrays are valid indices")
        return int(self._scalar())

    def __repr__(self):
        from ._copy_utils import asnumpy

        body = np.array2string(asnumpy(self), separator=", ", prefix="usm_ndarray(")
        return f"usm_ndarray({body}, dtype={self._dtype})" if self._dtype != np.float64 else f"usm_ndarray({body})"

    def __str__(self):
        from ._copy_utils import asnumpy

        return str(asnumpy(self))

    def to_device(self, target_device, /, *, stream=None):
        """Copy to another device (dpnp/tensor/_usmarray.pyx:1113-1191); a no-op for the same queue."""
        q = normalize_queue(device=target_device)
        if q == self._queue:
            return self
        from ._copy_utils import asnumpy, from_numpy

        return from_numpy(asnumpy(self), sycl_queue=q)

    # -------------------------------------------------------------- indexing
    def __getitem__(self, key):
        from ._slicing import basic_slice_meta

        shape, strides, offset, adv = basic_slice_meta(key, self._shape, self._strides)
        if adv:
            raise NotImplementedError("advanced (integer/boolean array) indexing is outside the elementwise/reduction path")
        return self._like(self._ptr + offset * self._dtype.itemsize, shape, strides)

    def __setitem__(self, key, value):
        from ._copy_utils import _assign_into

        if not (self._flags & FLAG_W):
            raise ValueError("Can not modify read-only array.")
        _assign_into(self[key], value)

    # ------------------------------------------------------------- operators
    def _ew(self, name):
        from . import _elementwise_funcs as ef

        return getattr(ef, name)

    def __add__(self, o): return self._ew("add")(self, o)
    def __radd__(self, o): return self._ew("add")(o, self)
    def __iadd__(self, o): return self._ew("add")._inplace_op(self, o)
    def __sub__(self, o): return self._ew("subtract")(self, o)
    def __rsub__(self, o): return self._ew("subtract")(o, self)
    def __isub__(self, o): return self._ew("subtract")._inplace_op(self, o)
    def __mul__(self, o): return self._ew("multiply")(self, o)
    def __rmul__(self, o): return self._ew("multiply")(o, self)
    def __imul__(self, o): return self._ew("multiply")._inplace_op(self, o)
    def __truediv__(self, o): return self._ew("divide")(self, o)
    def __rtruediv__(self, o): return self._ew("divide")(o, self)
    def __itruediv__(self, o): return self._ew("divide")._inplace_op(self, o)
    def __pow__(self, o): return self._ew("pow")(self, o)
    def __rpow__(self, o): return self._ew("pow")(o, self)
    def __neg__(self): return self._ew("negative")(self)
    def __pos__(self): return self._ew("positive")(self)
    def __abs__(self): return self._ew("abs")(self)
    def __lt__(self, o): return self._ew("less")(self, o)
    def __le__(self, o): return self._ew("less_equal")(self, o)
    def __gt__(self, o): return self._ew("greater")(self, o)
    def __ge__(self, o): return self._ew("greater_equal")(self, o)
    def __eq__(self, o): return self._ew("equal")(self, o)
    def __ne__(self, o): return self._ew("not_equal")(self, o)
    def __and__(self, o): return self._ew("bitwise_and")(self, o)
    def __rand__(self, o): return self._ew("bitwise_and")(o, self)
    def __iand__(self, o): return self._ew("bitwise_and")._inplace_op(self, o)
    def __or__(self, o): return self._ew("bitwise_or")(self, o)
    def __ror__(self, o): return self._ew("bitwise_or")(o, self)
    def __ior__(self, o): return self._ew("bitwise_or")._inplace_op(self, o)
    def __xor__(self, o): return self._ew("bitwise_xor")(self, o)
    def __rxor__(self, o): return self._ew("bitwise_xor")(o, self)
    def __ixor__(self, o): return self._ew("bitwise_xor")._inplace_op(self, o)
    def __invert__(self): return self._ew("bitwise_invert")(self)
    def __lshift__(self, o): return self._ew("bitwise_left_shift")(self, o)
    def __rlshift__(self, o): return self._ew("bitwise_left_shift")(o, self)
    def __ilshift__(self, o): return self._ew("bitwise_left_shift")._inplace_op(self, o)
    def __rshift__(self, o): return self._ew("bitwise_right_shift")(self, o)
    def __rrshift__(self, o): return self._ew("bitwise_right_shift")(o, self)
    def __irshift__(self, o): return self._ew("bitwise_right_shift")._inplace_op(self, o)
    def __floordiv__(self, o): return self._ew("floor_divide")(self, o)
    def __rfloordiv__(self, o): return self._ew("floor_divide")(o, self)
    def __ifloordiv__(self, o): return self._ew("floor_divide")._inplace_op(self, o)
    def __mod__(self, o): return self._ew("remainder")(self, o)
    def __rmod__(self, o): return self._ew("remainder")(o, self)
    def __imod__(self, o): return self._ew("remainder")._inplace_op(self, o)

    __hash__ = None
