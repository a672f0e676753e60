"""Python face of the native ``_tensor_elementwise_impl`` module of the reference
(dpnp/tensor/libtensor/source/tensor_elementwise.cpp:42-45 and one file per op,
e.g. source/elementwise_functions/add.cpp:188-241): for every operation
``_<op>(src[, src2], dst, sycl_queue, depends=[])``, ``_<op>_result_type(dtype[, dtype2])``
and ``_<op>_inplace(lhs, rhs, sycl_queue, depends=[])``, plus ``_divide_by_scalar``
(true_divide.cpp:494).  Validation, kernel choice and launch happen in
libdpnp_b200 (dpb_unary_ufunc / dpb_binary_ufunc / dpb_binary_inplace_ufunc).
"""

from __future__ import annotations

import ctypes as C
import sys

import numpy as np

from .. import _lib
from .._lib import BINARY_OPS, UNARY_OPS, check, lib
from ._tensor_impl import _check_queue, _events, _stream


_nat = _lib.native


def _make_unary(name, op):
    if _nat is not None:
        nat_unary = _nat.unary

        def call(src, dst, sycl_queue, depends=()):
            dev = sycl_queue.device
            if src._queue.device != dev or dst._queue.device != dev:
                _check_queue(sycl_queue, src, dst)
            nat_unary(op, src._core(), dst._core(), sycl_queue._stream)
            return _events(sycl_queue)
    else:
        def call(src, dst, sycl_queue, depends=()):
            _check_queue(sycl_queue, src, dst)
            ds, ks = src._descriptor()
            dd, kd = dst._descriptor()
            check(lib.dpb_unary_ufunc(op, C.byref(ds), C.byref(dd), _stream(sycl_queue)))
            return _events(sycl_queue)

    cache = {}

    def result_type(dtype):
        try:
            return cache[dtype]
        except (KeyError, TypeError):
            pass
        try:
            t = lib.dpb_unary_result_type(op, _lib.typenum_of(dtype))
        except TypeError:
            return None
        res = None if t < 0 else _lib.dtype_of(t)
        try:
            cache[dtype] = res
        except TypeError:
            pass
        return res

    call.__name__ = f"_{name}"
    result_type.__name__ = f"_{name}_result_type"
    return call, result_type


def _make_binary(name, op):
    if _nat is not None:
        nat_binary, nat_inplace = _nat.binary, _nat.binary_inplace

        def call(src1, src2, dst, sycl_queue, depends=()):
            dev = sycl_queue.device
            if src1._queue.device != dev or src2._queue.device != dev or dst._queue.device != dev:
                _check_queue(sycl_queue, src1, src2, dst)
            nat_binary(op, src1._core(), src2._core(), dst._core(), sycl_queue._stream)
            return _events(sycl_queue)
    else:
        def call(src1, src2, dst, sycl_queue, depends=()):
            _check_queue(sycl_queue, src1, src2, dst)
            d1, k1 = src1._descriptor()
            d2, k2 = src2._descriptor()
            dd, kd = dst._descriptor()
            check(lib.dpb_binary_ufunc(op, C.byref(d1), C.byref(d2), C.byref(dd), _stream(sycl_queue)))
            return _events(sycl_queue)

    cache = {}

    def result_type(dtype1, dtype2):
        try:
            return cache[(dtype1, dtype2)]
        except (KeyError, TypeError):
            pass
        try:
            t = lib.dpb_binary_result_type(op, _lib.typenum_of(dtype1), _lib.typenum_of(dtype2))
        except TypeError:
            return None
        res = None if t < 0 else _lib.dtype_of(t)
        try:
            cache[(dtype1, dtype2)] = res
        except TypeError:
            pass
        return res

    if _nat is not None:
        def inplace(lhs, rhs, sycl_queue, depends=()):
            _check_queue(sycl_queue, lhs, rhs)
            nat_inplace(op, lhs._core(), rhs._core(), sycl_queue._stream)
            return _events(sycl_queue)
    else:
        def inplace(lhs, rhs, sycl_queue, depends=()):
            _check_queue(sycl_queue, lhs, rhs)
            dl, kl = lhs._descriptor()
            dr, kr = rhs._descriptor()
            check(lib.dpb_binary_inplace_ufunc(op, C.byref(dl), C.byref(dr), _stream(sycl_queue)))
            return _events(sycl_queue)

    call.__name__ = f"_{name}"
    result_type.__name__ = f"_{name}_result_type"
    inplace.__name__ = f"_{name}_inplace"
    return call, result_type, inplace


_mod = sys.modules[__name__]
for _n, _op in UNARY_OPS.items():
    _c, _r = _make_unary(_n, _op)
    setattr(_mod, f"_{_n}", _c)
    setattr(_mod, f"_{_n}_result_type", _r)
for _n, _op in BINARY_OPS.items():
    _c, _r, _i = _make_binary(_n, _op)
    setattr(_mod, f"_{_n}", _c)
    setattr(_mod, f"_{_n}_result_type", _r)
    setattr(_mod, f"_{_n}_inplace", _i)


def _divide_by_scalar(src, scalar, dst, sycl_queue, depends=()):
    _check_queue(sycl_queue, src, dst)
    if _nat is not None:
        _nat.divide_by_scalar(src._core(), float(scalar), dst._core(), sycl_queue._stream)
        return _events(sycl_queue)
    ds, ks = src._descriptor()
    dd, kd = dst._descriptor()
    check(lib.dpb_divide_by_scalar(C.byref(ds), float(scalar), C.byref(dd), _stream(sycl_queue)))
    return _events(sycl_queue)
