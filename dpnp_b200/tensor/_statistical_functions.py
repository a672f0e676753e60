"""mean over axes: a sum in the result type followed by an in-place division by
the number of reduced elements (dpnp/tensor/_statistical_functions.py:166-270); var and std:
the two-pass composition of :38-163 and :273-380 (mean, deviations, squares, sum, division by
``n - correction``, and for std a square root), every step one kernel of this library."""

from __future__ import annotations

from . import _tensor_elementwise_impl as tei
from . import _tensor_impl as ti
from . import _tensor_reductions_impl as tri
from ._copy_utils import _empty, astype
from ._manipulation_functions import broadcast_to, normalize_axis_tuple, permute_dims, reshape
from ._type_utils import DEFAULT_FP
from ._usmarray import usm_ndarray


def mean(x, axis=None, keepdims=False):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    nd = x.ndim
    if axis is None:
        axis = tuple(range(nd))
    if not isinstance(axis, (tuple, list)):
        axis = (axis,)
    axis = normalize_axis_tuple(axis, nd, "axis")
    perm = [i for i in range(nd) if i not in axis]
    nelems = 1
    for i in axis:
        nelems *= x.shape[i]
    sum_nd = len(axis)
    perm = perm + list(axis)
    arr = permute_dims(x, perm)
    res_shape = arr.shape[: nd - sum_nd]
    q = x.sycl_queue
    res_dt = x.dtype if x.dtype.kind in "fc" else DEFAULT_FP
    if sum_nd == 0:
        return astype(x, res_dt, copy=True)
    res = _empty(res_shape, res_dt, q, "C", x.usm_type)
    if tri._sum_over_axis_dtype_supported(x.dtype, res_dt):
        tri._sum_over_axis(arr, sum_nd, res, sycl_queue=q)
    else:
        tmp = _empty(arr.shape, res_dt, q, "C", x.usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(arr, tmp, q)
        tri._sum_over_axis(tmp, sum_nd, res, sycl_queue=q)
    if keepdims:
        inv_perm = sorted(range(nd), key=lambda d: perm[d])
        res = permute_dims(reshape(res, tuple(res_shape) + (1,) * sum_nd), inv_perm)
    tei._divide_by_scalar(res, nelems, res, sycl_queue=q)
    return res


def _var_impl(x, axis, correction, keepdims):
    nd = x.ndim
    if axis is None:
        axis = tuple(range(nd))
    if not isinstance(axis, (tuple, list)):
        axis = (axis,)
    axis = normalize_axis_tuple(axis, nd, "axis")
    perm = [i for i in range(nd) if i not in axis]
    nelems = 1
    for i in axis:
        nelems *= x.shape[i]
    red_nd = len(axis)
    perm = perm + list(axis)
    q = x.sycl_queue
    res_dt = x.dtype if x.dtype.kind == "f" else DEFAULT_FP
    if x.dtype != res_dt:
        buf = _empty(x.shape, res_dt, q, "C", x.usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(x, buf, q)
    else:
        buf = x
    buf2 = permute_dims(buf, perm)
    res_shape = tuple(buf2.shape[: nd - red_nd])
    inv_perm = sorted(range(nd), key=lambda d: perm[d])
    if red_nd == 0:
        mean_ary = _empty(buf.shape, res_dt, q, "C", x.usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(buf, mean_ary, q)
    else:
        mean_ary = _empty(res_shape, res_dt, q, "C", x.usm_type)
        tri._sum_over_axis(buf2, red_nd, mean_ary, sycl_queue=q)
        mean_ary = permute_dims(reshape(mean_ary, res_shape + (1,) * red_nd), inv_perm)
    tei._divide_by_scalar(mean_ary, nelems, mean_ary, sycl_queue=q)
    dev_ary = _empty(buf.shape, res_dt, q, "C", x.usm_type)
    if tuple(mean_ary.shape) != tuple(buf.shape):
        mean_ary = broadcast_to(mean_ary, buf.shape)
    tei._subtract(buf, mean_ary, dev_ary, sycl_queue=q)
    tei._square(dev_ary, dev_ary, sycl_queue=q)
    if red_nd == 0:
        res = dev_ary
    else:
        res = _empty(res_shape, res_dt, q, "C", x.usm_type)
        tri._sum_over_axis(permute_dims(dev_ary, perm), red_nd, res, sycl_queue=q)
        if keepdims:
            res = permute_dims(reshape(res, res_shape + (1,) * red_nd), inv_perm)
    div = max(nelems - correction, 0)
    if not div:
        div = float("nan")                 # no degrees of freedom left: NaN
    tei._divide_by_scalar(res, div, res, sycl_queue=q)
    return res


def _check_var_args(x, correction):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    if not isinstance(correction, (int, float)):
        raise TypeError(f"Expected a Python integer or float for `correction`, got {type(correction)}")
    if x.dtype.kind == "c":
        raise ValueError("variance and standard deviation are not defined for complex types")


def var(x, axis=None, correction=0.0, keepdims=False):
    """Variance over `axis` with `correction` degrees of freedom removed."""
    _check_var_args(x, correction)
    return _var_impl(x, axis, correction, keepdims)


def std(x, axis=None, correction=0.0, keepdims=False):
    """Standard deviation: the square root, in place, of :func:`var`."""
    _check_var_args(x, correction)
    res = _var_impl(x, axis, correction, keepdims)
    tei._sqrt(res, res, sycl_queue=x.sycl_queue)
    return res
