"""Reductions over axes: sum, prod, max, min, argmax, argmin.

Orchestration as in dpnp/tensor/_reduction.py of the reference: reduced axes are
permuted to the end (:158-163), the result type defaults to the accumulation
type (:166-172), unsupported (input, output) type pairs go through a cast to a
temporary (:250-290), ``keepdims`` is a reshape plus inverse permutation
(:292-295); max/min/argmax/argmin refuse zero-size reduced axes (:59-60,322-323)
and argmax/argmin accept an integer axis or None only (:309-316).
"""

from __future__ import annotations

import builtins

import numpy as np

from ..memory import ExecutionPlacementError
from . import _tensor_impl as ti
from . import _tensor_reductions_impl as tri
from ._copy_utils import _empty
from ._ctors import empty_like
from ._elementwise_common import _common_queue
from ._manipulation_functions import normalize_axis_tuple, permute_dims, reshape, squeeze
from ._type_utils import DEFAULT_FP, DEFAULT_INDEX, _default_accumulation_dtype
from ._usmarray import usm_ndarray


def _permute_reduced_last(x, axis, int_axis_only=False):
    nd = len(x._shape)
    if axis is None:
        axis = tuple(range(nd))
        return x, axis, list(axis)
    if type(axis) is int and -nd <= axis < nd:
        a = axis + nd if axis < 0 else axis
        if a == nd - 1:                     # already last: no view needed
            return x, (a,), list(range(nd))
        perm = [i for i in range(nd) if i != a]
        perm.append(a)
        return permute_dims(x, perm), (a,), perm
    if int_axis_only:
        if not isinstance(axis, (int, np.integer)):
            raise TypeError("'axis' argument expected to have type 'int' or be `None`, "
                            f"got type {type(axis)}")
        axis = (axis,)
    elif not isinstance(axis, (tuple, list)):
        axis = (axis,)
    axis = normalize_axis_tuple(axis, nd, "axis")
    perm = [i for i in range(nd) if i not in axis] + list(axis)
    if perm == list(range(nd)):
        return x, axis, perm
    return permute_dims(x, perm), axis, perm


def _check_out(x, out, res_dt, res_shape, axis, keepdims, exec_q):
    """Validate `out`; returns (array to write, array the caller gave after squeezing)."""
    if not isinstance(out, usm_ndarray):
        raise TypeError(f"output array must be of usm_ndarray type, got {type(out)}")
    if not out.flags.writable:
        raise ValueError("provided `out` array is read-only")
    if keepdims:
        final_shape = tuple(1 if i in axis else s for i, s in enumerate(x.shape))
    else:
        final_shape = res_shape
    if out.shape != final_shape:
        raise ValueError("The shape of input and output arrays are inconsistent. "
                         f"Expected output shape is {final_shape}, got {out.shape}")
    if res_dt != out.dtype:
        raise ValueError(f"Output array of type {res_dt} is needed, got {out.dtype}")
    if _common_queue((exec_q, out.sycl_queue)) is None:
        raise ExecutionPlacementError("Input and output allocation queues are not compatible")
    if keepdims:
        out = squeeze(out, axis=axis)
    return out


def _restore_dims(out, res_shape, red_nd, perm, nd):
    res_shape = tuple(res_shape) + (1,) * red_nd
    inv_perm = sorted(range(nd), key=lambda d: perm[d])
    return permute_dims(reshape(out, res_shape), inv_perm)


def _reduction_over_axis(x, axis, dtype, keepdims, out, _reduction_fn, _dtype_supported,
                         _default_reduction_type_fn):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    nd = x.ndim
    arr, axis, perm = _permute_reduced_last(x, axis)
    red_nd = len(axis)
    res_shape = arr.shape[: nd - red_nd]
    q = x.sycl_queue
    inp_dt = x.dtype
    res_dt = _default_reduction_type_fn(inp_dt) if dtype is None else np.dtype(dtype)
    res_usm_type = x.usm_type
    implemented = _dtype_supported(inp_dt, res_dt, res_usm_type, q)
    if dtype is None and not implemented:
        raise RuntimeError("Automatically determined reduction data type does not have direct implementation")
    orig_out = out
    if out is not None:
        out = _check_out(x, out, res_dt, res_shape, axis, keepdims, q)
        orig_out = out
        if ti._array_overlap(x, out) and implemented:
            out = empty_like(out)
    else:
        out = _empty(res_shape, res_dt, q, "C", res_usm_type)

    if red_nd == 0:
        ti._copy_usm_ndarray_into_usm_ndarray(arr, out, q)
    elif implemented:
        _reduction_fn(arr, red_nd, out, sycl_queue=q)
    elif _dtype_supported(res_dt, res_dt, res_usm_type, q):
        tmp = _empty(arr.shape, res_dt, q, "C", res_usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(arr, tmp, q)
        _reduction_fn(tmp, red_nd, out, sycl_queue=q)
    else:
        buf_dt = _default_reduction_type_fn(inp_dt)
        tmp = _empty(arr.shape, buf_dt, q, "C", res_usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(arr, tmp, q)
        tmp_res = _empty(res_shape, buf_dt, q, "C", res_usm_type)
        _reduction_fn(tmp, red_nd, tmp_res, sycl_queue=q)
        ti._copy_usm_ndarray_into_usm_ndarray(tmp_res, out, q)
    if orig_out is not None and orig_out is not out:
        ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, q)
        out = orig_out
    if keepdims:
        out = _restore_dims(out, res_shape, red_nd, perm, nd)
    return out


def _comparison_over_axis(x, axis, keepdims, out, _reduction_fn):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    nd = x.ndim
    arr, axis, perm = _permute_reduced_last(x, axis)
    red_nd = len(axis)
    if builtins.any(arr.shape[i] == 0 for i in range(nd - red_nd, nd)):
        raise ValueError("reduction cannot be performed over zero-size axes")
    res_shape = arr.shape[: nd - red_nd]
    q = x.sycl_queue
    res_dt = x.dtype
    orig_out = out
    if out is not None:
        out = _check_out(x, out, res_dt, res_shape, axis, keepdims, q)
        orig_out = out
        if ti._array_overlap(x, out):
            out = empty_like(out)
    else:
        out = _empty(res_shape, res_dt, q, "C", x.usm_type)
    if red_nd == 0:
        ti._copy_usm_ndarray_into_usm_ndarray(arr, out, q)
    else:
        _reduction_fn(arr, red_nd, out, sycl_queue=q)
    if orig_out is not None and orig_out is not out:
        ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, q)
        out = orig_out
    if keepdims:
        out = _restore_dims(out, res_shape, red_nd, perm, nd)
    return out


def _search_over_axis(x, axis, keepdims, out, _reduction_fn):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    nd = x.ndim
    arr, axis, perm = _permute_reduced_last(x, axis, int_axis_only=True)
    red_nd = len(axis)
    if builtins.any(arr.shape[i] == 0 for i in range(nd - red_nd, nd)):
        raise ValueError("reduction cannot be performed over zero-size axes")
    res_shape = arr.shape[: nd - red_nd]
    q = x.sycl_queue
    res_dt = DEFAULT_INDEX
    orig_out = out
    if out is not None:
        out = _check_out(x, out, res_dt, res_shape, axis, keepdims, q)
        orig_out = out
        if ti._array_overlap(x, out) and red_nd > 0:
            out = empty_like(out)
    else:
        out = _empty(res_shape, res_dt, q, "C", x.usm_type)
    if red_nd == 0:
        ti._full_usm_ndarray(0, out, q)
        return out
    _reduction_fn(arr, red_nd, out, sycl_queue=q)
    if orig_out is not None and orig_out is not out:
        ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, q)
        out = orig_out
    if keepdims:
        out = _restore_dims(out, res_shape, red_nd, perm, nd)
    return out


def sum(x, /, *, axis=None, dtype=None, keepdims=False, out=None):
    """Sum of the elements over the given axes."""
    return _reduction_over_axis(x, axis, dtype, keepdims, out, tri._sum_over_axis,
                                tri._sum_over_axis_dtype_supported, _default_accumulation_dtype)


def prod(x, /, *, axis=None, dtype=None, keepdims=False, out=None):
    """Product of the elements over the given axes."""
    return _reduction_over_axis(x, axis, dtype, keepdims, out, tri._prod_over_axis,
                                tri._prod_over_axis_dtype_supported, _default_accumulation_dtype)


def _default_accumulation_dtype_fp_types(inp_dt):
    """Result type of a reduction that exists for floating types only: the input's own type,
    the default floating type for bool and integers (dpnp/tensor/_type_utils.py:955-972)."""
    if inp_dt.kind in "biu":
        res = DEFAULT_FP
        return res if np.can_cast(inp_dt, res) else np.dtype("f8")
    if inp_dt.kind == "f":
        return inp_dt
    raise ValueError("function not defined for complex types")


def _to_fp_operand(x):
    """bool and integer input of a floating-only reduction is converted to the result type first
    (the reference's kernels convert each element on load: the values are the same)."""
    if isinstance(x, usm_ndarray) and x.dtype.kind in "biu":
        from ._copy_utils import astype
        return astype(x, _default_accumulation_dtype_fp_types(x.dtype))
    return x


def logsumexp(x, /, *, axis=None, dtype=None, keepdims=False, out=None):
    """log(sum(exp(x))) over the given axes, merged pairwise with logaddexp
    (dpnp/tensor/_reduction.py:515-577)."""
    x = _to_fp_operand(x)
    return _reduction_over_axis(x, axis, dtype, keepdims, out, tri._logsumexp_over_axis,
                                tri._logsumexp_over_axis_dtype_supported,
                                _default_accumulation_dtype_fp_types)


def reduce_hypot(x, /, *, axis=None, dtype=None, keepdims=False, out=None):
    """sqrt(sum(x**2)) over the given axes, merged pairwise with hypot
    (dpnp/tensor/_reduction.py:707-768)."""
    x = _to_fp_operand(x)
    return _reduction_over_axis(x, axis, dtype, keepdims, out, tri._hypot_over_axis,
                                tri._hypot_over_axis_dtype_supported,
                                _default_accumulation_dtype_fp_types)


def count_nonzero(x, /, *, axis=None, keepdims=False, out=None):
    """Number of non-zero elements: the sum of the truth values in the index type
    (dpnp/tensor/_reduction.py:472-512)."""
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    if x.dtype != np.bool_:
        from ._copy_utils import astype
        x = astype(x, np.bool_, copy=False)
    return sum(x, axis=axis, dtype=DEFAULT_INDEX, keepdims=keepdims, out=out)


def max(x, /, *, axis=None, keepdims=False, out=None):
    """Maximum over the given axes (NaN propagates)."""
    return _comparison_over_axis(x, axis, keepdims, out, tri._max_over_axis)


def min(x, /, *, axis=None, keepdims=False, out=None):
    """Minimum over the given axes (NaN propagates)."""
    return _comparison_over_axis(x, axis, keepdims, out, tri._min_over_axis)


def argmax(x, /, *, axis=None, keepdims=False, out=None):
    """Index of the first maximum along an axis (flattened when axis is None)."""
    return _search_over_axis(x, axis, keepdims, out, tri._argmax_over_axis)


def argmin(x, /, *, axis=None, keepdims=False, out=None):
    """Index of the first minimum along an axis (flattened when axis is None)."""
    return _search_over_axis(x, axis, keepdims, out, tri._argmin_over_axis)


def _boolean_reduction(x, axis, keepdims, fn):
    """all/any: the array is first reduced to its truth values, then max/min of
    booleans is logical or/and (the reference has dedicated kernels,
    source/reductions/reduction_over_axis.hpp:1053-1303; the results are the same)."""
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    from ._copy_utils import astype
    b = x if x.dtype == np.bool_ else astype(x, np.bool_)
    if b.size == 0 or any_zero_axis(b, axis):
        # empty reductions: all -> True, any -> False
        from ._ctors import full
        nd = b.ndim
        axes = tuple(range(nd)) if axis is None else normalize_axis_tuple(
            axis if isinstance(axis, (tuple, list)) else (axis,), nd)
        shape = tuple((1 if i in axes else s) for i, s in enumerate(b.shape) if keepdims or i not in axes)
        return full(shape, fn is min, dtype=np.bool_, sycl_queue=x.sycl_queue)
    return fn(b, axis=axis, keepdims=keepdims)


def any_zero_axis(x, axis):
    nd = x.ndim
    axes = range(nd) if axis is None else normalize_axis_tuple(
        axis if isinstance(axis, (tuple, list)) else (axis,), nd)
    for i in axes:
        if x.shape[i] == 0:
            return True
    return False


def all(x, /, *, axis=None, keepdims=False):
    """True where every element along the axes is non-zero."""
    return _boolean_reduction(x, axis, keepdims, min)


def any(x, /, *, axis=None, keepdims=False):
    """True where some element along the axes is non-zero."""
    return _boolean_reduction(x, axis, keepdims, max)
