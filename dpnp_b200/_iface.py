"""Functions of the public NumPy-compatible API other than the ufunc objects:
array creation, views, copies, reductions, ``where`` and helpers.

Keyword handling follows the reference wrappers: ``sum``/``prod``
(dpnp/dpnp_iface_mathematical.py:4910-5010 with the accumulation type of :96-103),
``max``/``min``/``mean`` (dpnp/dpnp_iface_statistics.py:1039-1207), ``argmax``/``argmin``
(dpnp/dpnp_iface_searching.py:69-158), ``where`` (:386-475), the ``out`` handling of
dpnp/dpnp_utils/dpnp_utils_reduction.py:35-52 and ``get_result_array``
(dpnp/dpnp_iface.py:495-540): ``initial``/``where`` are not supported, an ``out`` of
another type receives the result with an unsafe cast.
"""

from __future__ import annotations

import numpy as np

from . import _fusion
from . import tensor as dpt
from .dpnp_array import dpnp_array
from .tensor import _tensor_impl as ti
from .tensor._type_utils import DEFAULT_FP, _default_accumulation_dtype
from .tensor._usmarray import usm_ndarray


def _wrap(x):
    return dpnp_array._create_from_usm_ndarray(x) if isinstance(x, usm_ndarray) else x


def is_supported_array_type(a):
    return isinstance(a, (dpnp_array, usm_ndarray))


def get_usm_ndarray(a):
    """The tensor-level array behind `a` (dpnp/dpnp_iface.py:543-571)."""
    if isinstance(a, dpnp_array):
        return a._array_obj
    if isinstance(a, usm_ndarray):
        return a
    raise TypeError(f"An array must be any of supported type, but got {type(a)}")


def get_usm_ndarray_or_scalar(a):
    return a if isinstance(a, (bool, int, float, complex, np.generic)) else get_usm_ndarray(a)


def check_limitations(initial=None, where=True, **kw):
    """Raise NotImplementedError for keywords the device path does not implement."""
    if initial is not None:
        raise NotImplementedError(f"initial keyword argument is only supported with its default value, got {initial}")
    if where is not True:
        raise NotImplementedError(f"where keyword argument is only supported with its default value, got {where}")


def asnumpy(a, order="C"):
    """Copy to a NumPy array (dpnp/dpnp_iface.py:107-140)."""
    if isinstance(a, (dpnp_array, usm_ndarray)):
        return np.asarray(dpt.asnumpy(get_usm_ndarray(a)), order=order)
    return np.asarray(a, order=order)


def default_float_type(device=None, sycl_queue=None):
    """Default floating type of the device: float64 (dpnp/dpnp_iface.py:309-344)."""
    return DEFAULT_FP.type


def are_same_logical_tensors(a, b):
    return ti._same_logical_tensors(get_usm_ndarray(a), get_usm_ndarray(b))


def copyto(dst, src, casting="same_kind", where=True):
    if where is not True:
        raise NotImplementedError("where keyword is not supported")
    dst_usm = get_usm_ndarray(dst)
    if isinstance(src, (dpnp_array, usm_ndarray)):
        src = get_usm_ndarray(src)
        if not np.can_cast(src.dtype, dst_usm.dtype, casting=casting):
            raise TypeError(f"Cannot cast from {src.dtype} to {dst_usm.dtype} according to the rule '{casting}'")
    dst_usm[...] = src


def get_result_array(a, out=None, casting="safe"):
    if out is None:
        return _wrap(a)
    out_arr = _wrap(out)
    a_usm = get_usm_ndarray(a)
    if a is out or ti._same_logical_tensors(a_usm, out_arr._array_obj):
        return out_arr
    if out_arr.shape != a_usm.shape:
        raise ValueError(f"Output array of shape {a_usm.shape} is needed, got {out_arr.shape}.")
    copyto(out_arr, a_usm, casting=casting)
    return out_arr


# ---------------------------------------------------------------- creation
def _creation(fn):
    def wrapped(*args, like=None, **kwargs):
        if like is not None:
            raise NotImplementedError("like keyword is not supported")
        args = [get_usm_ndarray(a) if isinstance(a, dpnp_array) else a for a in args]
        return _wrap(fn(*args, **kwargs))
    wrapped.__name__ = fn.__name__
    wrapped.__doc__ = fn.__doc__
    return wrapped


empty = _creation(dpt.empty)
zeros = _creation(dpt.zeros)
ones = _creation(dpt.ones)
arange = _creation(dpt.arange)


def linspace(start, stop, /, num, *, dtype=None, device=None, usm_type=None, sycl_queue=None, endpoint=True,
             retstep=False, axis=0):
    """Evenly spaced numbers over an interval (dpnp/dpnp_iface_arraycreation.py: linspace); scalar
    end points only on this path."""
    if retstep or axis != 0:
        raise NotImplementedError("linspace with retstep or axis is not provided by this path")
    return _wrap(dpt.linspace(start, stop, num, dtype=dtype, device=device, usm_type=usm_type or "device",
                              sycl_queue=sycl_queue, endpoint=endpoint))


def from_dlpack(x, /, *, device=None, copy=None):
    """Array sharing the memory of a DLPack producer (dpnp/dpnp_iface.py: from_dlpack)."""
    return _wrap(dpt.from_dlpack(x, device=device, copy=copy))

empty_like = _creation(dpt.empty_like)
zeros_like = _creation(dpt.zeros_like)
ones_like = _creation(dpt.ones_like)


def full(shape, fill_value, *, dtype=None, order="C", like=None, device=None, usm_type=None, sycl_queue=None):
    fv = get_usm_ndarray(fill_value) if isinstance(fill_value, dpnp_array) else fill_value
    return _wrap(dpt.full(shape, fv, dtype=dtype, order=order, device=device, usm_type=usm_type,
                          sycl_queue=sycl_queue))


def full_like(a, /, fill_value, *, dtype=None, order="K", device=None, usm_type=None, sycl_queue=None):
    return _wrap(dpt.full_like(get_usm_ndarray(a), fill_value, dtype=dtype, order=order, device=device,
                               usm_type=usm_type, sycl_queue=sycl_queue))


def asarray(a, dtype=None, order=None, *, device=None, usm_type=None, sycl_queue=None, copy=None, like=None):
    if isinstance(a, dpnp_array):
        a = a._array_obj
    return _wrap(dpt.asarray(a, dtype=dtype, order=order or "K", device=device, usm_type=usm_type,
                             sycl_queue=sycl_queue, copy=copy))


def ascontiguousarray(a, dtype=None, *, like=None, device=None, usm_type=None, sycl_queue=None):
    """C-contiguous array with the contents of `a`; `a` itself when it already is one
    (dpnp/dpnp_iface_arraycreation.py: ascontiguousarray)."""
    if like is not None:
        raise NotImplementedError("like keyword is not supported")
    if isinstance(a, (dpnp_array, usm_ndarray)):
        u = get_usm_ndarray(a)
        if u.flags.c_contiguous and (dtype is None or np.dtype(dtype) == u.dtype):
            return _wrap(u)
    return asarray(a, dtype=dtype, order="C", device=device, usm_type=usm_type, sycl_queue=sycl_queue)


def array(a, dtype=None, *, copy=True, order="K", subok=False, ndmin=0, like=None, device=None,
          usm_type=None, sycl_queue=None):
    if subok or like is not None:
        raise NotImplementedError("subok/like keywords are not supported")
    r = asarray(a, dtype=dtype, order=order, device=device, usm_type=usm_type, sycl_queue=sycl_queue,
                copy=True if copy else None)
    if ndmin > r.ndim:
        r = r.reshape((1,) * (ndmin - r.ndim) + r.shape)
    return r


def astype(x, dtype, /, *, order="K", casting="unsafe", copy=True, device=None):
    return _wrap(dpt.astype(get_usm_ndarray(x), dtype, order=order, casting=casting, copy=copy))


def copy(a, order="K", subok=False):
    return _wrap(dpt.copy(get_usm_ndarray(a), order=order))


# ------------------------------------------------------------------- views
def transpose(a, axes=None):
    a = _wrap(a)
    return a.transpose() if axes is None else a.transpose(*axes)


def reshape(a, /, shape=None, order="C", *, newshape=None, copy=None):
    if shape is None:
        shape = newshape
    if shape is None:
        raise TypeError("reshape() missing 1 required positional argument: 'shape'")
    if order is None:
        order = "C"
    if order in ("A", "a"):
        u = get_usm_ndarray(a)
        order = "F" if (u.flags.f_contiguous and not u.flags.c_contiguous) else "C"
    return _wrap(dpt.reshape(get_usm_ndarray(a), shape, order=order, copy=copy))


def broadcast_to(a, /, shape, subok=False):
    return _wrap(dpt.broadcast_to(get_usm_ndarray(a), shape))


def expand_dims(a, axis):
    return _wrap(dpt.expand_dims(get_usm_ndarray(a), axis))


def squeeze(a, /, axis=None):
    return _wrap(dpt.squeeze(get_usm_ndarray(a), axis))


def ravel(a, order="C"):
    return reshape(a, -1, order=order)


# -------------------------------------------------------------- reductions
def _wrap_reduction_call(usm_a, out, fn, res_dt, **kwargs):
    input_out = out
    usm_out = None
    if out is not None:
        if not is_supported_array_type(out):
            raise TypeError(f"An array must be any of supported type, but got {type(out)}")
        out_usm = get_usm_ndarray(out)
        # the tensor layer wants the exact result type; other types get the
        # result through a cast afterwards
        usm_out = out_usm if out_usm.dtype == res_dt else None
    kwargs["out"] = usm_out
    res = fn(usm_a, **kwargs)
    return get_result_array(res, input_out, casting="unsafe")


def _reduction_res_dt(a, dtype):
    return _default_accumulation_dtype(a.dtype) if dtype is None else np.dtype(dtype)


def _sharded(a):
    """The hook of a sharded array (dpnp_b200.sharded.ShardedArray), else None."""
    return None if type(a) is dpnp_array else getattr(a, "__dpnp_sharded__", None)


def sum(a, axis=None, dtype=None, out=None, keepdims=False, initial=None, where=True):
    check_limitations(initial=initial, where=where)
    sh = _sharded(a)
    if sh is not None:
        return sh("sum", axis, dtype, keepdims, out)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.sum, _reduction_res_dt(usm_a, dtype), axis=axis,
                                dtype=dtype, keepdims=keepdims)


def prod(a, axis=None, dtype=None, out=None, keepdims=False, initial=None, where=True):
    check_limitations(initial=initial, where=where)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.prod, _reduction_res_dt(usm_a, dtype), axis=axis,
                                dtype=dtype, keepdims=keepdims)


def max(a, axis=None, out=None, keepdims=False, initial=None, where=True):
    check_limitations(initial=initial, where=where)
    sh = _sharded(a)
    if sh is not None:
        return sh("max", axis, None, keepdims, out)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.max, usm_a.dtype, axis=axis, keepdims=keepdims)


def min(a, axis=None, out=None, keepdims=False, initial=None, where=True):
    check_limitations(initial=initial, where=where)
    sh = _sharded(a)
    if sh is not None:
        return sh("min", axis, None, keepdims, out)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.min, usm_a.dtype, axis=axis, keepdims=keepdims)


amax, amin = max, min


def argmax(a, axis=None, out=None, *, keepdims=False):
    sh = _sharded(a)
    if sh is not None:
        if out is not None:
            raise NotImplementedError("out= is not supported for reductions of sharded arrays")
        return sh("argmax", axis, keepdims)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.argmax, np.dtype("i8"), axis=axis, keepdims=keepdims)


def argmin(a, axis=None, out=None, *, keepdims=False):
    sh = _sharded(a)
    if sh is not None:
        if out is not None:
            raise NotImplementedError("out= is not supported for reductions of sharded arrays")
        return sh("argmin", axis, keepdims)
    usm_a = get_usm_ndarray(a)
    return _wrap_reduction_call(usm_a, out, dpt.argmin, np.dtype("i8"), axis=axis, keepdims=keepdims)


def mean(a, /, axis=None, dtype=None, out=None, keepdims=False, *, where=True):
    check_limitations(where=where)
    sh = _sharded(a)
    if sh is not None:
        if out is not None or dtype is not None:
            raise NotImplementedError("out= and dtype= are not supported for the mean of a sharded array")
        return sh("mean", axis, keepdims)
    res = dpt.mean(get_usm_ndarray(a), axis=axis, keepdims=keepdims)
    if dtype is not None:
        res = dpt.astype(res, dtype)
    return get_result_array(res, out, casting="unsafe")


def _cumulative(fn, a, axis, dtype, out, include_initial=False, flatten=True):
    """cumsum/cumprod flatten a multi-dimensional input when no axis is given
    (dpnp/dpnp_iface_mathematical.py:1100-1180); `out` of another type is filled by a cast
    (dpnp/dpnp_utils/dpnp_utils_reduction.py:35-52)."""
    if not is_supported_array_type(a):
        raise TypeError(f"An array must be any of supported type, but got {type(a)}")
    usm_a = get_usm_ndarray(a)
    if flatten and usm_a.ndim > 1 and axis is None:
        usm_a = dpt.reshape(usm_a, (-1,))
    res_dt = np.dtype(dtype) if dtype is not None else None
    usm_out = None
    if out is not None:
        if not is_supported_array_type(out):
            raise TypeError(f"An array must be any of supported type, but got {type(out)}")
        usm_out = get_usm_ndarray(out)
        from .tensor._reduction import _default_accumulation_dtype_fp_types
        default = _default_accumulation_dtype_fp_types if fn is dpt.cumulative_logsumexp \
            else _default_accumulation_dtype
        if usm_out.dtype != (res_dt if res_dt is not None else default(usm_a.dtype)):
            usm_out = None                       # filled below by a cast
    res = fn(usm_a, axis=axis, dtype=dtype, include_initial=include_initial, out=usm_out)
    return get_result_array(res, out, casting="unsafe")


def cumsum(a, axis=None, dtype=None, out=None):
    return _cumulative(dpt.cumulative_sum, a, axis, dtype, out)


def cumprod(a, axis=None, dtype=None, out=None):
    return _cumulative(dpt.cumulative_prod, a, axis, dtype, out)


def cumlogsumexp(x, /, *, axis=None, dtype=None, include_initial=False, out=None):
    return _cumulative(dpt.cumulative_logsumexp, x, axis, dtype, out, include_initial, flatten=False)


def cumulative_sum(x, /, *, axis=None, dtype=None, out=None, include_initial=False):
    return _cumulative(dpt.cumulative_sum, x, axis, dtype, out, include_initial, flatten=False)


def cumulative_prod(x, /, *, axis=None, dtype=None, out=None, include_initial=False):
    return _cumulative(dpt.cumulative_prod, x, axis, dtype, out, include_initial, flatten=False)


def count_nonzero(a, axis=None, *, keepdims=False, out=None):
    """Number of non-zero elements over `axis` (dpnp/dpnp_iface_counting.py:49-105)."""
    return get_result_array(dpt.count_nonzero(get_usm_ndarray(a), axis=axis, keepdims=keepdims), out)


def logsumexp(x, /, *, axis=None, out=None, dtype=None, keepdims=False):
    """log(sum(exp(x))) over `axis` (dpnp/dpnp_iface_trigonometric.py: logsumexp)."""
    res = dpt.logsumexp(get_usm_ndarray(x), axis=axis, dtype=dtype, keepdims=keepdims)
    return get_result_array(res, out, casting="same_kind")


def reduce_hypot(x, /, *, axis=None, out=None, dtype=None, keepdims=False):
    """sqrt(sum(x**2)) over `axis` (dpnp/dpnp_iface_trigonometric.py: reduce_hypot)."""
    res = dpt.reduce_hypot(get_usm_ndarray(x), axis=axis, dtype=dtype, keepdims=keepdims)
    return get_result_array(res, out, casting="same_kind")


def _spread(name, a, axis, dtype, out, ddof, keepdims, where, mean, correction):
    """Shared keyword handling of var/std (dpnp/dpnp_iface_statistics.py:1470-1668 and
    :1665-1860): `correction` is the array-API spelling of `ddof`; complex input and a
    caller-supplied `mean` are outside this path."""
    if not is_supported_array_type(a):
        raise TypeError(f"An array must be any of supported type, but got {type(a)}")
    check_limitations(where=where)
    if correction is not None:
        if ddof != 0:
            raise ValueError("ddof and correction can't be provided simultaneously.")
        ddof = correction
    if not isinstance(ddof, (int, float)):
        raise TypeError(f"An integer or float is required, but got {type(ddof)}")
    if mean is not None:
        raise NotImplementedError(f"{name} with a precomputed mean is not provided by this path")
    fn = dpt.var if name == "var" else dpt.std
    result = get_result_array(fn(get_usm_ndarray(a), axis=axis, correction=ddof, keepdims=keepdims), out)
    if dtype is not None and out is None:
        result = result.astype(dtype, casting="same_kind")
    return result


def var(a, /, axis=None, dtype=None, out=None, ddof=0, keepdims=False, *, where=True, mean=None,
        correction=None):
    return _spread("var", a, axis, dtype, out, ddof, keepdims, where, mean, correction)


def std(a, /, axis=None, dtype=None, out=None, ddof=0, keepdims=False, *, where=True, mean=None,
        correction=None):
    return _spread("std", a, axis, dtype, out, ddof, keepdims, where, mean, correction)


def where(condition, x=None, y=None, /, *, order="K", out=None):
    """Elements from `x` where `condition` holds, else from `y`
    (dpnp/dpnp_iface_searching.py:386-475; the one-argument form is not on this path)."""
    missing = (x is None, y is None).count(True)
    if missing == 1:
        raise ValueError("Must provide both 'x' and 'y' or neither.")
    if missing == 2:
        raise NotImplementedError("where(condition) alone (nonzero) is not provided by the elementwise path")
    if _fusion.is_traced(condition, x, y):         # inside a function that is being fused
        return _fusion.trace_where(condition, x, y, out)
    cond = get_usm_ndarray(condition)
    xu = get_usm_ndarray_or_scalar(x)
    yu = get_usm_ndarray_or_scalar(y)
    res = dpt.where(cond, xu, yu, order=order, out=None if out is None else get_usm_ndarray(out))
    return get_result_array(res, out)


def flip(m, axis=None):
    return _wrap(dpt.flip(get_usm_ndarray(m), axis=axis))


def all(a, /, axis=None, out=None, keepdims=False, *, where=True):
    check_limitations(where=where)
    return get_result_array(dpt.all(get_usm_ndarray(a), axis=axis, keepdims=keepdims), out)


def any(a, /, axis=None, out=None, keepdims=False, *, where=True):
    check_limitations(where=where)
    return get_result_array(dpt.any(get_usm_ndarray(a), axis=axis, keepdims=keepdims), out)
