"""where(condition, x1, x2): elements from x1 where the condition holds, else from x2.

Semantics of dpnp/tensor/_search_functions.py:109-415 of the reference: the
result type is the promotion of x1 and x2 (Python scalars are weak), x1 and x2
are cast to it before the kernel runs, the condition may have any type
(non-zero is true), result layout follows the order-"K" rule over all three
inputs, ``out`` must match shape and type exactly and may not partially
overlap an input.
"""

from __future__ import annotations

import numpy as np

from ..memory import ExecutionPlacementError
from . import _tensor_impl as ti
from ._copy_utils import _empty, _empty_like_orderK, _empty_like_triple_orderK
from ._ctors import asarray, empty_like
from ._elementwise_common import _coerce_usm_type, _common_queue, _scalar_to_array
from ._manipulation_functions import _broadcast_shape_impl, broadcast_to
from ._type_utils import _get_dtype, _get_shape, _is_weak_dtype, _promote_weak, _validate_dtype
from ._usmarray import usm_ndarray


def _where_result_type(dt1, dt2):
    res = np.promote_types(dt1, dt2)
    return res


def where(condition, x1, x2, /, *, order="K", out=None):
    if not isinstance(condition, usm_ndarray):
        raise TypeError(f"Expecting dpnp.tensor.usm_ndarray type, got {type(condition)}")
    if order not in ("K", "C", "F", "A"):
        order = "K"
    queues = [condition.sycl_queue] + [o.sycl_queue for o in (x1, x2) if isinstance(o, usm_ndarray)]
    exec_q = _common_queue(queues)
    if exec_q is None:
        raise ExecutionPlacementError(
            "Execution placement can not be unambiguously inferred from input arguments.")
    out_usm_type = _coerce_usm_type(
        [condition.usm_type] + [o.usm_type for o in (x1, x2) if isinstance(o, usm_ndarray)])
    x1_shape, x2_shape = _get_shape(x1), _get_shape(x2)
    if not all(isinstance(s, (tuple, list)) for s in (x1_shape, x2_shape)):
        raise TypeError("Shape of arguments can not be inferred. Arguments are expected to be "
                        "lists, tuples, or both")
    try:
        res_shape = _broadcast_shape_impl([condition.shape, x1_shape, x2_shape])
    except ValueError:
        raise ValueError("operands could not be broadcast together with shapes "
                         f"{condition.shape}, {x1_shape}, and {x2_shape}") from None
    x1_dtype, x2_dtype = _get_dtype(x1), _get_dtype(x2)
    if not all(_validate_dtype(o) for o in (x1_dtype, x2_dtype)):
        raise ValueError("Operands have unsupported data types")
    if _is_weak_dtype(x1_dtype) and _is_weak_dtype(x2_dtype):
        # two Python scalars: default type of the wider kind
        k = max(x1_dtype.kind_num, x2_dtype.kind_num)
        x1_dtype = x2_dtype = {0: np.dtype("?"), 1: np.dtype("i8"), 2: np.dtype("f8"),
                               3: np.dtype("c16")}[k]
    elif _is_weak_dtype(x1_dtype):
        x1_dtype = _promote_weak(x1_dtype, x2_dtype, False)
    elif _is_weak_dtype(x2_dtype):
        x2_dtype = _promote_weak(x2_dtype, x1_dtype, False)
    out_dtype = _where_result_type(x1_dtype, x2_dtype)

    orig_out = out
    if out is not None:
        if not isinstance(out, usm_ndarray):
            raise TypeError(f"output array must be of usm_ndarray type, got {type(out)}")
        if not out.flags.writable:
            raise ValueError("provided `out` array is read-only")
        if out.shape != res_shape:
            raise ValueError("The shape of input and output arrays are inconsistent. "
                             f"Expected output shape is {res_shape}, got {out.shape}")
        if out_dtype != out.dtype:
            raise ValueError(f"Output array of type {out_dtype} is needed, got {out.dtype}")
        if _common_queue((exec_q, out.sycl_queue)) is None:
            raise ExecutionPlacementError("Input and output allocation queues are not compatible")
        if ti._array_overlap(condition, out) and not ti._same_logical_tensors(condition, out):
            out = empty_like(out)
        for o, dt in ((x1, x1_dtype), (x2, x2_dtype)):
            if (isinstance(o, usm_ndarray) and out is orig_out and dt == out_dtype
                    and ti._array_overlap(o, out) and not ti._same_logical_tensors(o, out)):
                out = empty_like(out)

    if order == "A":
        arrs = [condition] + [o for o in (x1, x2) if isinstance(o, usm_ndarray)]
        order = "F" if all(a.flags.f_contiguous for a in arrs) else "C"
    if not isinstance(x1, usm_ndarray):
        x1 = _scalar_to_array(x1, x1_dtype, exec_q)
    if not isinstance(x2, usm_ndarray):
        x2 = _scalar_to_array(x2, x2_dtype, exec_q)

    if condition.size == 0:
        if out is not None:
            return orig_out
        return _empty(res_shape, out_dtype, exec_q, "F" if order == "F" else "C", out_usm_type)

    def _cast(x):
        if x.dtype == out_dtype:
            return x
        b = _empty_like_orderK(x, out_dtype) if order == "K" else empty_like(x, dtype=out_dtype, order=order)
        ti._copy_usm_ndarray_into_usm_ndarray(x, b, exec_q)
        return b

    x1, x2 = _cast(x1), _cast(x2)
    if out is None:
        if order == "K":
            out = _empty_like_triple_orderK(condition, x1, x2, out_dtype, res_shape, out_usm_type, exec_q)
        else:
            out = _empty(res_shape, out_dtype, exec_q, order, out_usm_type)
    cond_b = broadcast_to(condition, res_shape) if condition.shape != res_shape else condition
    x1 = broadcast_to(x1, res_shape) if x1.shape != res_shape else x1
    x2 = broadcast_to(x2, res_shape) if x2.shape != res_shape else x2
    ti._where(cond_b, x1, x2, out, sycl_queue=exec_q)
    if orig_out is not None and orig_out is not out:
        ti._copy_usm_ndarray_into_usm_ndarray(out, orig_out, exec_q)
        out = orig_out
    return out
