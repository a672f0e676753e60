"""cumulative_sum / cumulative_prod / cumulative_logsumexp: argument handling of the
reference's ``_accumulate_common`` (dpnp/tensor/_accumulation.py:47-262): the scanned axis is
moved last, the result type is the default accumulation type unless ``dtype`` is given, an
``out`` that overlaps the input is filled through a temporary, and input types without a direct
kernel are converted first."""

from __future__ import annotations

import numpy as np

from ..memory import ExecutionPlacementError
from . import _tensor_accumulation_impl as tai
from . import _tensor_impl as ti
from ._copy_utils import _empty
from ._ctors import empty_like
from ._elementwise_common import _common_queue
from ._manipulation_functions import normalize_axis_tuple, permute_dims, reshape, squeeze
from ._reduction import _default_accumulation_dtype_fp_types
from ._type_utils import _default_accumulation_dtype
from ._usmarray import usm_ndarray


def _accumulate_common(x, axis, dtype, include_initial, out, _accumulate_fn, _include_initial_fn,
                       _dtype_supported, _default_type_fn):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected dpnp.tensor.usm_ndarray, got {type(x)}")
    appended_axis = False
    if x.ndim == 0:
        x = reshape(x, (1,))
        appended_axis = True
    nd = x.ndim
    if axis is None:
        if nd > 1:
            raise ValueError(f"`axis` cannot be `None` for array of dimension `{nd}`")
        axis = 0
    else:
        axis = normalize_axis_tuple((axis,), nd, "axis")[0]
    sh = tuple(x.shape)
    res_sh = sh[:axis] + (sh[axis] + 1,) + sh[axis + 1:] if include_initial else sh
    a1 = axis + 1
    if a1 == nd:
        perm = list(range(nd))
        arr = x
    else:
        perm = [i for i in range(nd) if i != axis] + [axis]
        arr = permute_dims(x, perm)
    q = x.sycl_queue
    inp_dt = x.dtype
    res_dt = _default_type_fn(inp_dt) if dtype is None else np.dtype(dtype)
    implemented = _dtype_supported(inp_dt, res_dt)
    if dtype is None and not implemented:
        raise RuntimeError("Automatically determined accumulation data type does not have direct implementation")
    orig_out = out
    if out is not None:
        if not isinstance(out, usm_ndarray):
            raise TypeError(f"output array must be of usm_ndarray type, got {type(out)}")
        if not out.flags.writable:
            raise ValueError("provided `out` array is read-only")
        out_sh = tuple(out.shape)
        if appended_axis and not include_initial:
            out = reshape(out, (1,) + out_sh)
            orig_out = out
            final_res_sh = res_sh[1:]
        else:
            final_res_sh = res_sh
        if out_sh != final_res_sh:
            raise ValueError("The shape of input and output arrays are inconsistent. "
                             f"Expected output shape is {final_res_sh}, got {out_sh}")
        if res_dt != out.dtype:
            raise ValueError(f"Output array of type {res_dt} is needed, got {out.dtype}")
        if _common_queue((q, out.sycl_queue)) is None:
            raise ExecutionPlacementError("Input and output allocation queues are not compatible")
        if a1 != nd:
            out = permute_dims(out, perm)
            orig_out = out
        if ti._array_overlap(x, out) and implemented:
            out = empty_like(out)
    else:
        out = _empty(res_sh, res_dt, q, "C", x.usm_type)
        if a1 != nd:
            out = permute_dims(out, perm)

    def run(src, dst):
        if include_initial:
            _include_initial_fn(src, dst, sycl_queue=q)
        else:
            _accumulate_fn(src, 1, dst, sycl_queue=q)

    if implemented:
        run(arr, out)
        if not (orig_out is None or out is orig_out):
            ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, q)
            out = orig_out
    elif _dtype_supported(res_dt, res_dt):
        tmp = _empty(arr.shape, res_dt, q, "C", x.usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(arr, tmp, q)
        run(tmp, out)
    else:
        buf_dt = _default_type_fn(inp_dt)
        tmp = _empty(arr.shape, buf_dt, q, "C", x.usm_type)
        ti._copy_usm_ndarray_into_usm_ndarray(arr, tmp, q)
        tmp_res = _empty(res_sh, buf_dt, q, "C", x.usm_type)
        if a1 != nd:
            tmp_res = permute_dims(tmp_res, perm)
        run(tmp, tmp_res)
        ti._copy_usm_ndarray_into_usm_ndarray(tmp_res, out, q)
    if appended_axis:
        out = squeeze(out)
    if a1 != nd:
        inv_perm = sorted(range(nd), key=lambda d: perm[d])
        out = permute_dims(out, inv_perm)
    return out


def cumulative_sum(x, /, *, axis=None, dtype=None, include_initial=False, out=None):
    """Running sum along `axis` (dpnp/tensor/_accumulation.py:265-338)."""
    return _accumulate_common(x, axis, dtype, include_initial, out, tai._cumsum_over_axis,
                              tai._cumsum_final_axis_include_initial, tai._cumsum_dtype_supported,
                              _default_accumulation_dtype)


def cumulative_prod(x, /, *, axis=None, dtype=None, include_initial=False, out=None):
    """Running product along `axis` (dpnp/tensor/_accumulation.py:341-415)."""
    return _accumulate_common(x, axis, dtype, include_initial, out, tai._cumprod_over_axis,
                              tai._cumprod_final_axis_include_initial, tai._cumprod_dtype_supported,
                              _default_accumulation_dtype)


def cumulative_logsumexp(x, /, *, axis=None, dtype=None, include_initial=False, out=None):
    """Running log(sum(exp(x))) along `axis` (dpnp/tensor/_accumulation.py:418-490)."""
    if isinstance(x, usm_ndarray) and x.dtype.kind in "biu":
        from ._copy_utils import astype
        x = astype(x, _default_accumulation_dtype_fp_types(x.dtype))
    return _accumulate_common(x, axis, dtype, include_initial, out, tai._cumlogsumexp_over_axis,
                              tai._cumlogsumexp_final_axis_include_initial,
                              tai._cumlogsumexp_dtype_supported, _default_accumulation_dtype_fp_types)
