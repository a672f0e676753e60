"""``dpnp.ndarray``: the NumPy-compatible array of the public API.

A thin object over :class:`dpnp_b200.tensor.usm_ndarray`, as ``dpnp_array`` is in
the reference (dpnp/dpnp_array.py:99-160 constructor, :162-658 operators,
:660 ``_create_from_usm_ndarray``, :2051-2099 byte strides).  Strides are
reported in BYTES here and in elements on the underlying tensor.
"""

from __future__ import annotations

import numpy as np

from . import tensor as dpt
from .tensor._usmarray import usm_ndarray


def _unwrap(x):
    return x._array_obj if isinstance(x, dpnp_array) else x


class dpnp_array:
    """Multi-dimensional array on a CUDA device with NumPy semantics."""

    __array_priority__ = 200.0

    def __init__(self, shape, dtype=None, buffer=None, offset=0, strides=None, order="C",
                 device=None, usm_type="device", sycl_queue=None):
        if order is None:
            order = "C"
        if buffer is not None:
            buffer = _unwrap(buffer)
            dtype = buffer.dtype if dtype is None else np.dtype(dtype)
            if strides is not None:
                strides = tuple(s // dtype.itemsize for s in strides)
            self._array_obj = usm_ndarray(shape, dtype=dtype, strides=strides, buffer=buffer,
                                          offset=offset, order=order)
        else:
            from .memory import normalize_queue

            q = normalize_queue(sycl_queue, device)
            dtype = np.dtype("f8") if dtype is None else np.dtype(dtype)
            if strides is not None:
                strides = tuple(s // dtype.itemsize for s in strides)
            self._array_obj = usm_ndarray(shape, dtype=dtype, strides=strides, buffer=usm_type,
                                          offset=offset, order=order, buffer_ctor_kwargs={"queue": q})

    @staticmethod
    def _create_from_usm_ndarray(usm_ary):
        if not isinstance(usm_ary, usm_ndarray):
            raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(usm_ary)}")
        res = dpnp_array.__new__(dpnp_array)
        res._array_obj = usm_ary
        return res

    # -------------------------------------------------------------- protocol
    @property
    def __usm_ndarray__(self):
        return self._array_obj

    def get_array(self):
        """The underlying :class:`usm_ndarray`."""
        return self._array_obj

    def __dlpack__(self, **kwargs):
        return self._array_obj.__dlpack__(**kwargs)

    def __dlpack_device__(self):
        return self._array_obj.__dlpack_device__()

    @property
    def __cuda_array_interface__(self):
        return self._array_obj.__cuda_array_interface__

    # ------------------------------------------------------------ attributes
    @property
    def shape(self):
        return self._array_obj.shape

    @shape.setter
    def shape(self, newshape):
        self._array_obj.shape = newshape

    @property
    def strides(self):
        """Strides in bytes, as in NumPy."""
        item = self._array_obj.itemsize
        return tuple(s * item for s in self._array_obj.strides)

    @property
    def dtype(self):
        return self._array_obj.dtype

    @property
    def ndim(self):
        return self._array_obj.ndim

    @property
    def size(self):
        return self._array_obj.size

    @property
    def itemsize(self):
        return self._array_obj.itemsize

    @property
    def nbytes(self):
        return self._array_obj.nbytes

    @property
    def flags(self):
        return self._array_obj.flags

    @property
    def T(self):
        return self.transpose()

    @property
    def mT(self):
        return dpnp_array._create_from_usm_ndarray(self._array_obj.mT)

    @property
    def sycl_queue(self):
        return self._array_obj.sycl_queue

    @property
    def sycl_device(self):
        return self._array_obj.sycl_device

    @property
    def device(self):
        return self._array_obj.device

    @property
    def usm_type(self):
        return self._array_obj.usm_type

    @property
    def data(self):
        return self._array_obj.usm_data

    # ----------------------------------------------------------- conversions
    def asnumpy(self):
        return dpt.asnumpy(self._array_obj)

    def __array__(self, dtype=None, copy=None):
        raise TypeError(
            "Implicit conversion to a NumPy array is not allowed. Please use `.asnumpy()` to "
            "construct a NumPy array explicitly.")

    def __len__(self):
        return len(self._array_obj)

    def __bool__(self):
        return bool(self._array_obj)

    def __float__(self):
        return float(self._array_obj)

    def __int__(self):
        return int(self._array_obj)

    def __complex__(self):
        return complex(self._array_obj)

    def __index__(self):
        return self._array_obj.__index__()

    def item(self, *args):
        return self.asnumpy().item(*args)

    def tolist(self):
        return self.asnumpy().tolist()

    def __repr__(self):
        body = np.array2string(self.asnumpy(), separator=", ", prefix="array(")
        default = self.dtype in (np.dtype("f8"), np.dtype("i8"), np.dtype("?"), np.dtype("c16"))
        return f"array({body})" if default and self.size else f"array({body}, dtype={self.dtype})"

    def __str__(self):
        return str(self.asnumpy())

    # -------------------------------------------------------------- indexing
    def __getitem__(self, key):
        key = _unwrap(key)
        if isinstance(key, tuple):
            key = tuple(_unwrap(k) for k in key)
        return dpnp_array._create_from_usm_ndarray(self._array_obj[key])

    def __setitem__(self, key, val):
        key = _unwrap(key)
        if isinstance(key, tuple):
            key = tuple(_unwrap(k) for k in key)
        self._array_obj[key] = _unwrap(val)

    # ------------------------------------------------------------- operators
    def _fn(self, name):
        import dpnp_b200 as dpnp

        return getattr(dpnp, name)

    def __add__(self, o): return self._fn("add")(self, o)
    def __radd__(self, o): return self._fn("add")(o, self)
    def __iadd__(self, o): self._fn("add")(self, o, out=self); return self
    def __sub__(self, o): return self._fn("subtract")(self, o)
    def __rsub__(self, o): return self._fn("subtract")(o, self)
    def __isub__(self, o): self._fn("subtract")(self, o, out=self); return self
    def __mul__(self, o): return self._fn("multiply")(self, o)
    def __rmul__(self, o): return self._fn("multiply")(o, self)
    def __imul__(self, o): self._fn("multiply")(self, o, out=self); return self
    def __truediv__(self, o): return self._fn("divide")(self, o)
    def __rtruediv__(self, o): return self._fn("divide")(o, self)
    def __itruediv__(self, o): self._fn("divide")(self, o, out=self); return self
    def __pow__(self, o): return self._fn("power")(self, o)
    def __rpow__(self, o): return self._fn("power")(o, self)
    def __neg__(self): return self._fn("negative")(self)
    def __pos__(self): return self._fn("positive")(self)
    def __abs__(self): return self._fn("abs")(self)
    def __lt__(self, o): return self._fn("less")(self, o)
    def __le__(self, o): return self._fn("less_equal")(self, o)
    def __gt__(self, o): return self._fn("greater")(self, o)
    def __ge__(self, o): return self._fn("greater_equal")(self, o)
    def __eq__(self, o): return self._fn("equal")(self, o)
    def __ne__(self, o): return self._fn("not_equal")(self, o)
    def __and__(self, o): return self._fn("bitwise_and")(self, o)
    def __rand__(self, o): return self._fn("bitwise_and")(o, self)
    def __iand__(self, o): self._fn("bitwise_and")(self, o, out=self); return self
    def __or__(self, o): return self._fn("bitwise_or")(self, o)
    def __ror__(self, o): return self._fn("bitwise_or")(o, self)
    def __ior__(self, o): self._fn("bitwise_or")(self, o, out=self); return self
    def __xor__(self, o): return self._fn("bitwise_xor")(self, o)
    def __rxor__(self, o): return self._fn("bitwise_xor")(o, self)
    def __ixor__(self, o): self._fn("bitwise_xor")(self, o, out=self); return self
    def __invert__(self): return self._fn("invert")(self)
    def __lshift__(self, o): return self._fn("left_shift")(self, o)
    def __rlshift__(self, o): return self._fn("left_shift")(o, self)
    def __ilshift__(self, o): self._fn("left_shift")(self, o, out=self); return self
    def __rshift__(self, o): return self._fn("right_shift")(self, o)
    def __rrshift__(self, o): return self._fn("right_shift")(o, self)
    def __irshift__(self, o): self._fn("right_shift")(self, o, out=self); return self
    def __floordiv__(self, o): return self._fn("floor_divide")(self, o)
    def __rfloordiv__(self, o): return self._fn("floor_divide")(o, self)
    def __ifloordiv__(self, o): self._fn("floor_divide")(self, o, out=self); return self
    def __mod__(self, o): return self._fn("remainder")(self, o)
    def __rmod__(self, o): return self._fn("remainder")(o, self)
    def __imod__(self, o): self._fn("remainder")(self, o, out=self); return self

    __hash__ = None

    # --------------------------------------------------------------- methods
    def transpose(self, *axes):
        nd = self.ndim
        if nd <= 1:
            return self
        if len(axes) == 1 and (axes[0] is None or isinstance(axes[0], (tuple, list))):
            axes = axes[0]
        if not axes:
            axes = tuple(range(nd - 1, -1, -1))
        return dpnp_array._create_from_usm_ndarray(dpt.permute_dims(self._array_obj, axes))

    def reshape(self, *shape, order="C", copy=None):
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = shape[0]
        return self._fn("reshape")(self, shape, order=order, copy=copy)

    def astype(self, dtype, order="K", casting="unsafe", subok=True, copy=True, device=None):
        return self._fn("astype")(self, dtype, order=order, casting=casting, copy=copy)

    def copy(self, order="C"):
        return dpnp_array._create_from_usm_ndarray(dpt.copy(self._array_obj, order=order))

    def fill(self, value):
        self._array_obj[...] = _unwrap(value)

    def to_device(self, device):
        return dpnp_array._create_from_usm_ndarray(self._array_obj.to_device(device))

    def sum(self, axis=None, dtype=None, out=None, keepdims=False, initial=None, where=True):
        return self._fn("sum")(self, axis=axis, dtype=dtype, out=out, keepdims=keepdims,
                               initial=initial, where=where)

    def prod(self, axis=None, dtype=None, out=None, keepdims=False, initial=None, where=True):
        return self._fn("prod")(self, axis=axis, dtype=dtype, out=out, keepdims=keepdims,
                                initial=initial, where=where)

    def mean(self, axis=None, dtype=None, out=None, keepdims=False, *, where=True):
        return self._fn("mean")(self, axis=axis, dtype=dtype, out=out, keepdims=keepdims, where=where)

    def max(self, axis=None, out=None, keepdims=False, initial=None, where=True):
        return self._fn("max")(self, axis=axis, out=out, keepdims=keepdims, initial=initial, where=where)

    def min(self, axis=None, out=None, keepdims=False, initial=None, where=True):
        return self._fn("min")(self, axis=axis, out=out, keepdims=keepdims, initial=initial, where=where)

    def argmax(self, axis=None, out=None, *, keepdims=False):
        return self._fn("argmax")(self, axis=axis, out=out, keepdims=keepdims)

    def argmin(self, axis=None, out=None, *, keepdims=False):
        return self._fn("argmin")(self, axis=axis, out=out, keepdims=keepdims)
