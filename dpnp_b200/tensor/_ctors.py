"""Array creation (glue for the elementwise/reduction path).

Follows the creation functions of dpnp/tensor/_ctors.py (asarray :677, empty
:879, zeros :1127, ones, full :1517, arange :566, *_like): allocation comes from
the stream-ordered pool, initial values from fill kernels or a host staging copy.
"""

from __future__ import annotations

import builtins
import operator

import numpy as np

from .. import _lib
from ..memory import normalize_queue
from . import _tensor_impl as ti
from ._copy_utils import _empty, astype, from_numpy
from ._usmarray import _normalize_shape, usm_ndarray

_default_fp = np.dtype("f8")
_default_int = np.dtype("i8")


def _check_order(order):
    if not isinstance(order, str) or order.upper() not in ("C", "F"):
        raise ValueError("Unrecognized order keyword value, expecting 'F' or 'C'.")
    return order.upper()


def _check_usm_type(usm_type):
    if usm_type not in ("device", "shared", "host"):
        raise ValueError(f"Unrecognized value of usm_type={usm_type}, expected 'device', 'shared', or 'host'.")


def empty(shape, *, dtype=None, order="C", device=None, usm_type="device", sycl_queue=None):
    order = _check_order(order)
    _check_usm_type(usm_type)
    q = normalize_queue(sycl_queue, device)
    dtype = _default_fp if dtype is None else np.dtype(dtype)
    shape = _normalize_shape(shape)
    if len(shape) > _lib.MAX_ND:
        raise ValueError(f"arrays with more than {_lib.MAX_ND} dimensions are not supported")
    return _empty(shape, dtype, q, order, usm_type)


def zeros(shape, *, dtype=None, order="C", device=None, usm_type="device", sycl_queue=None):
    r = empty(shape, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue)
    if r.size:
        ti._zeros_usm_ndarray(r, r.sycl_queue)
    return r


def _dtype_of_scalar(v):
    if isinstance(v, (bool, np.bool_)):
        return np.dtype("?")
    if isinstance(v, (int, np.integer)):
        return _default_int if not isinstance(v, np.integer) else np.dtype(type(v))
    if isinstance(v, (float, np.floating)):
        return _default_fp if not isinstance(v, np.floating) else np.dtype(type(v))
    if isinstance(v, (complex, np.complexfloating)):
        return np.dtype("c16") if not isinstance(v, np.complexfloating) else np.dtype(type(v))
    raise TypeError(f"scalar of type {type(v)} is not supported")


def full(shape, fill_value, *, dtype=None, order="C", device=None, usm_type=None, sycl_queue=None):
    if isinstance(fill_value, usm_ndarray):
        if fill_value.size != 1:
            raise ValueError("fill_value must be a scalar or a one-element array")
        q = normalize_queue(sycl_queue, device) if (sycl_queue or device) else fill_value.sycl_queue
        dtype = fill_value.dtype if dtype is None else dtype
        r = empty(shape, dtype=dtype, order=order, usm_type=usm_type or fill_value.usm_type, sycl_queue=q)
        from ._copy_utils import _assign_into
        _assign_into(r, fill_value)
        return r
    if dtype is None:
        dtype = _dtype_of_scalar(fill_value)
    r = empty(shape, dtype=dtype, order=order, device=device, usm_type=usm_type or "device",
              sycl_queue=sycl_queue)
    if r.size:
        ti._full_usm_ndarray(fill_value, r, r.sycl_queue)
    return r


def ones(shape, *, dtype=None, order="C", device=None, usm_type="device", sycl_queue=None):
    return full(shape, 1, dtype=_default_fp if dtype is None else dtype, order=order, device=device,
                usm_type=usm_type, sycl_queue=sycl_queue)


def _like_kwargs(x, dtype, order, device, usm_type, sycl_queue):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected instance of dpt.usm_ndarray, got {type(x)}.")
    dtype = x.dtype if dtype is None else dtype
    usm_type = x.usm_type if usm_type is None else usm_type
    if device is None and sycl_queue is None:
        sycl_queue = x.sycl_queue
    order = order.upper() if isinstance(order, str) else order
    if order not in ("C", "F", "A", "K"):
        raise ValueError("Unrecognized order keyword value, expecting 'K', 'A', 'F', or 'C'.")
    if order == "A":
        order = "F" if (x.flags.f_contiguous and not x.flags.c_contiguous) else "C"
    return dtype, order, device, usm_type, sycl_queue


def empty_like(x, /, *, dtype=None, order="K", device=None, usm_type=None, sycl_queue=None):
    dtype, order, device, usm_type, sycl_queue = _like_kwargs(x, dtype, order, device, usm_type, sycl_queue)
    if order == "K":
        from ._copy_utils import _empty_like_orderK
        return _empty_like_orderK(x, np.dtype(dtype), usm_type, normalize_queue(sycl_queue, device))
    return empty(x.shape, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue)


def zeros_like(x, /, *, dtype=None, order="K", device=None, usm_type=None, sycl_queue=None):
    r = empty_like(x, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue)
    if r.size:
        ti._full_usm_ndarray(0, r, r.sycl_queue)
    return r


def ones_like(x, /, *, dtype=None, order="K", device=None, usm_type=None, sycl_queue=None):
    r = empty_like(x, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue)
    if r.size:
        ti._full_usm_ndarray(1, r, r.sycl_queue)
    return r


def full_like(x, /, fill_value, *, dtype=None, order="K", device=None, usm_type=None, sycl_queue=None):
    r = empty_like(x, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue)
    if r.size:
        ti._full_usm_ndarray(fill_value, r, r.sycl_queue)
    return r


def asarray(obj, /, *, dtype=None, device=None, copy=None, usm_type=None, sycl_queue=None, order="K"):
    """Convert `obj` to a device array (arrays pass through unless a cast or copy is needed)."""
    if hasattr(obj, "__usm_ndarray__") and not isinstance(obj, usm_ndarray):
        obj = obj.__usm_ndarray__
    if isinstance(obj, usm_ndarray):
        x = obj
        if device is not None or sycl_queue is not None:
            x = x.to_device(normalize_queue(sycl_queue, device))
        if dtype is not None and np.dtype(dtype) != x.dtype:
            if copy is False:
                raise ValueError("asarray(..., copy=False) would need a cast")
            return astype(x, dtype, order=order, copy=True)
        if copy:
            return astype(x, x.dtype, order=order, copy=True)
        if order in ("C", "F") and not x.flags[order]:
            return astype(x, x.dtype, order=order, copy=True)
        return x
    if copy is False:
        raise ValueError("Converting a host object to a device array requires a copy")
    if isinstance(obj, (bool, int, float, complex)) and dtype is None:
        dtype = _dtype_of_scalar(obj)
    np_ary = np.asarray(obj, dtype=dtype)
    if np_ary.dtype == object:
        raise TypeError("object arrays are not supported")
    if np_ary.dtype.kind in "SUV":
        raise TypeError(f"data type {np_ary.dtype} is not supported")
    if order in ("C", "c"):
        np_ary = np.ascontiguousarray(np_ary)
    elif order in ("F", "f"):
        np_ary = np.asfortranarray(np_ary)
    return from_numpy(np_ary, device=device, usm_type=usm_type or "device", sycl_queue=sycl_queue)


def _get_arange_length(start, stop, step):
    """Number of elements of arange: ceil((stop - start) / step), computed in Python numbers
    (dpnp/tensor/_ctors.py:549-563)."""
    span = stop - start
    if type(step) in (int, float) and type(span) in (int, float):
        import math
        return math.ceil(span / step)
    tmp = span / step
    return tmp.real.__ceil__() if tmp.imag == 0 else min(tmp.real.__ceil__(), tmp.imag.__ceil__())


def arange(start, /, stop=None, step=1, *, dtype=None, device=None, usm_type="device", sycl_queue=None):
    """Evenly spaced values in a half-open interval, written on the device
    (dpnp/tensor/_ctors.py:566-674): element i is ``first + i * (second - first)`` in the
    array's own arithmetic, with first and second rounded to the array's type."""
    if stop is None:
        stop, start = start, 0
    if step is None:
        step = 1
    _check_usm_type(usm_type)
    for v in (start, stop, step):
        if not isinstance(v, (int, float, np.integer, np.floating)) or isinstance(v, (bool, np.bool_)):
            raise ValueError("start, stop, and step must be Python scalars")
    q = normalize_queue(sycl_queue, device)
    is_bool = dtype is not None and np.dtype(dtype) == np.bool_
    if dtype is None:
        dt = _default_fp if any(isinstance(v, (float, np.floating)) for v in (start, stop, step)) else _default_int
    else:
        dt = np.dtype("i1") if is_bool else np.dtype(dtype)
    if dt.kind not in "iuf":
        raise ValueError(f"arange does not produce arrays of type {dt}")
    try:
        sh = builtins.max(int(_get_arange_length(start, stop, step)), 0)
    except (TypeError, ZeroDivisionError, OverflowError):
        sh = 0
    if is_bool and sh > 2:
        raise ValueError("no fill-function for boolean data type")
    res = _empty((sh,), dt, q, "C", usm_type)
    if sh:
        sc = dt.type
        with np.errstate(all="ignore"):
            first = sc(start)
            if sh > 1:
                second = sc(start + step)
                stepv = sc(np.int64(second) - np.int64(first)) if dt.kind == "u" else sc(second - first)
            else:
                stepv = sc(1)
        a0, a1 = np.array([first], dtype=dt), np.array([stepv], dtype=dt)
        _lib.check(_lib.lib.dpb_linspace_step(_lib.typenum_of(dt), res._ptr, sh, a0.ctypes.data, a1.ctypes.data,
                                              q.stream))
    return astype(res, np.bool_) if is_bool else res


def linspace(start, stop, /, num, *, dtype=None, device=None, endpoint=True, sycl_queue=None,
             usm_type="device"):
    """`num` evenly spaced values from start to stop, written on the device
    (dpnp/tensor/_ctors.py:1340-1440): integer types are produced in the default floating type
    and converted at the end."""
    _check_usm_type(usm_type)
    if endpoint not in (True, False):
        raise TypeError("endpoint keyword argument must be of boolean type")
    num = operator.index(num)
    if num < 0:
        raise ValueError("Number of points must be non-negative")
    for v in (start, stop):
        if not isinstance(v, (bool, int, float, np.integer, np.floating, np.bool_)):
            raise ValueError("start and stop must be Python scalars.")
    q = normalize_queue(sycl_queue, device)
    if dtype is None:
        dt = _default_fp
    else:
        dt = np.dtype(dtype)
    int_dt = None
    if dt.kind in "biu":
        int_dt = dt if dtype is not None else None
        dt = _default_fp
    if dt.kind != "f":
        raise ValueError(f"linspace does not produce arrays of type {dt}")
    res = _empty((num,), dt, q, "C", usm_type)
    if num:
        a0, a1 = np.array([float(start)], dtype=dt), np.array([float(stop)], dtype=dt)
        _lib.check(_lib.lib.dpb_linspace_affine(_lib.typenum_of(dt), res._ptr, num, a0.ctypes.data,
                                                a1.ctypes.data, int(bool(endpoint)), q.stream))
    return res if int_dt is None else astype(res, int_dt)
