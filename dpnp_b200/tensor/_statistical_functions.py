"""mean over axes: a sum in the result type followed by an in-place division by
the number of reduced elements (dpnp/tensor/_statistical_functions.py:166-270)."""

from __future__ import annotations

from . import _tensor_elementwise_impl as tei
from . import _tensor_impl as ti
from . import _tensor_reductions_impl as tri
from ._copy_utils import _empty, astype
from ._manipulation_functions import normalize_axis_tuple, permute_dims, reshape
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
