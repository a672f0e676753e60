"""Host<->device transfers, copies, casts and order-"K" allocation.

Semantics follow dpnp/tensor/_copy_utils.py of the reference: ``asnumpy`` /
``from_numpy`` (host staging), ``copy``/``astype`` (:993-..), the order-K
allocation rules ``_empty_like_orderK`` and its two/three-input forms
(:782-989), and assignment with overlap handling (:634-690,710-779).
"""

from __future__ import annotations

import builtins
import ctypes as C

import numpy as np

from .. import _lib
from .._lib import check, lib
from ..memory import normalize_queue
from . import _tensor_impl as ti
from ._usmarray import usm_ndarray


def _empty(shape, dtype, queue, order="C", usm_type="device"):
    """Uninitialised dense array; `shape` is a validated tuple/list of extents."""
    if type(dtype) is not np.dtype:
        dtype = np.dtype(dtype)
    _lib.typenum_of(dtype)
    return usm_ndarray._new_dense(shape if type(shape) is tuple else tuple(shape), dtype, queue,
                                  _lib.FLAG_F if order in ("F", "f") else _lib.FLAG_C, usm_type)


def asnumpy(x) -> np.ndarray:
    """Copy a device array to a new NumPy array (synchronises the array's stream)."""
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray, got {type(x)}")
    q = x.sycl_queue
    if x.size == 0:
        return np.empty(x.shape, dtype=x.dtype)
    src = x
    if not x.flags.c_contiguous:
        src = _empty(x.shape, x.dtype, q)
        ti._copy_usm_ndarray_into_usm_ndarray(x, src, q)
    out = np.empty(x.shape, dtype=x.dtype)
    q.activate()
    check(lib.dpb_memcpy(C.c_void_p(out.ctypes.data), C.c_void_p(src._ptr), out.nbytes, 1,
                         C.c_void_p(q.stream)))
    q.wait()
    return out


to_numpy = asnumpy


def _copy_from_numpy_into(dst: usm_ndarray, np_ary: np.ndarray) -> None:
    """dst[...] = np_ary (broadcast and cast on the host, one H2D copy)."""
    q = dst.sycl_queue
    src = np.ascontiguousarray(np.broadcast_to(np_ary, dst.shape), dtype=dst.dtype) \
        if np_ary.dtype == dst.dtype else \
        np.ascontiguousarray(np.broadcast_to(np_ary, dst.shape)).astype(dst.dtype, casting="unsafe")
    if dst.size == 0:
        return
    q.activate()
    if dst.flags.c_contiguous:
        check(lib.dpb_memcpy(C.c_void_p(dst._ptr), C.c_void_p(src.ctypes.data), src.nbytes, 0,
                             C.c_void_p(q.stream)))
        q.wait()  # the host buffer must outlive the copy
        return
    tmp = _empty(dst.shape, dst.dtype, q)
    check(lib.dpb_memcpy(C.c_void_p(tmp._ptr), C.c_void_p(src.ctypes.data), src.nbytes, 0,
                         C.c_void_p(q.stream)))
    ti._copy_usm_ndarray_into_usm_ndarray(tmp, dst, q)
    q.wait()


def from_numpy(np_ary, /, *, device=None, usm_type="device", sycl_queue=None) -> usm_ndarray:
    """New device array with the contents (and order) of a NumPy array."""
    np_ary = np.asarray(np_ary)
    q = normalize_queue(sycl_queue, device)
    _lib.typenum_of(np_ary.dtype)
    order = "F" if (np_ary.flags.f_contiguous and not np_ary.flags.c_contiguous) else "C"
    res = _empty(np_ary.shape, np_ary.dtype, q, order=order, usm_type=usm_type)
    if order == "F":
        _copy_from_numpy_into(res.T, np_ary.T)
    else:
        _copy_from_numpy_into(res, np_ary)
    return res


def _orderK_perm(arrays, ndim):
    sts = [list(a.strides) + [0] * (ndim - a.ndim) for a in arrays]
    shs = [list(a.shape) + [0] * (ndim - a.ndim) for a in arrays]
    perm = sorted(range(ndim),
                  key=lambda d: tuple(builtins.abs(st[d]) if sh[d] > 1 else 0 for st, sh in zip(sts, shs)),
                  reverse=True)
    return perm, sts


def _empty_like_orderK_multi(arrays, dt, res_shape, usm_type, queue):
    """Order-"K" result allocation for 1..3 inputs."""
    res_shape = tuple(res_shape)
    arrays = list(arrays)
    # inputs of lower rank than the result do not influence the layout when
    # all remaining inputs already have the result shape
    full = [a for a in arrays if a.shape == res_shape]
    lower = [a for a in arrays if a.ndim < len(res_shape)]
    if full and lower and len(full) + len(lower) == len(arrays):
        arrays = full
    if len(arrays) == 1 and arrays[0].shape == res_shape:
        x = arrays[0]
        if x.flags.c_contiguous or x.size <= 1:
            return _empty(res_shape, dt, queue, "C", usm_type)
        if x.flags.f_contiguous:
            return _empty(res_shape, dt, queue, "F", usm_type)
    else:
        if builtins.any(a.flags.c_contiguous for a in arrays):
            return _empty(res_shape, dt, queue, "C", usm_type)
        if builtins.all(a.flags.f_contiguous for a in arrays):
            return _empty(res_shape, dt, queue, "F", usm_type)
    ndim = len(res_shape)
    perm, sts = _orderK_perm(arrays, ndim)
    inv_perm = sorted(range(ndim), key=lambda i: perm[i])
    sh_sorted = tuple(res_shape[i] for i in perm)
    r = _empty(sh_sorted, dt, queue, "C", usm_type)
    sorted_sts = [[st[i] for i in perm] for st in sts]
    if ndim and builtins.max(builtins.min(s) for s in sorted_sts) < 0:
        sl = tuple(slice(None, None, -1) if builtins.all(s[i] < 0 for s in sorted_sts) else slice(None)
                   for i in range(ndim))
        r = r[sl]
    from ._manipulation_functions import permute_dims
    return permute_dims(r, inv_perm)


def _empty_like_orderK(x, dt, usm_type=None, dev=None):
    return _empty_like_orderK_multi([x], dt, x.shape, usm_type or x.usm_type, dev or x.sycl_queue)


def _empty_like_pair_orderK(x1, x2, dt, res_shape, usm_type, dev):
    return _empty_like_orderK_multi([x1, x2], dt, res_shape, usm_type, dev)


def _empty_like_triple_orderK(x1, x2, x3, dt, res_shape, usm_type, dev):
    return _empty_like_orderK_multi([x1, x2, x3], dt, res_shape, usm_type, dev)


def copy(x, /, *, order="K"):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray, got {type(x)}")
    return astype(x, x.dtype, order=order, copy=True)


def astype(x, newdtype, /, *, order="K", casting="unsafe", copy=True, device=None):
    if not isinstance(x, usm_ndarray):
        raise TypeError(f"Expected usm_ndarray, got {type(x)}")
    if order not in ("C", "F", "A", "K", "c", "f", "a", "k"):
        raise ValueError("Unrecognized value of the order keyword. Recognized values are 'A', 'C', 'F', or 'K'")
    order = order.upper()
    newdtype = np.dtype(newdtype)
    _lib.typenum_of(newdtype)
    if not np.can_cast(x.dtype, newdtype, casting=casting):
        raise TypeError(f"Can not cast from {x.dtype} to {newdtype} according to rule {casting}.")
    c, f = x.flags.c_contiguous, x.flags.f_contiguous
    needs_copy = copy or x.dtype != newdtype
    if not needs_copy and (order == "K" or (order == "A" and (c or f)) or (order == "C" and c) or
                           (order == "F" and f)):
        return x
    if order == "A":
        order = "F" if (f and not c) else "C"
    q = x.sycl_queue
    if order == "K":
        r = _empty_like_orderK(x, newdtype)
    else:
        r = _empty(x.shape, newdtype, q, order, x.usm_type)
    ti._copy_usm_ndarray_into_usm_ndarray(x, r, q)
    return r


def _assign_into(dst: usm_ndarray, value) -> None:
    """dst[...] = value for arrays, NumPy arrays and Python scalars."""
    from ._manipulation_functions import broadcast_to

    q = dst.sycl_queue
    if isinstance(value, usm_ndarray):
        if value.sycl_queue.device != q.device:
            value = value.to_device(q)
        if value.shape != dst.shape:
            try:
                value = broadcast_to(value, dst.shape)
            except ValueError:
                raise ValueError(
                    f"Shape of array to assign from, {value.shape}, can not be broadcast to {dst.shape}") from None
        if dst.size == 0:
            return
        if ti._array_overlap(value, dst) and not ti._same_logical_tensors(value, dst):
            value = astype(value, value.dtype, order="C", copy=True)
        ti._copy_usm_ndarray_into_usm_ndarray(value, dst, q)
        return
    if hasattr(value, "__usm_ndarray__"):
        return _assign_into(dst, value.__usm_ndarray__)
    if isinstance(value, (bool, int, float, complex, np.generic)):
        if dst.size:
            ti._full_usm_ndarray(value, dst, q)
        return
    _copy_from_numpy_into(dst, np.asarray(value))
