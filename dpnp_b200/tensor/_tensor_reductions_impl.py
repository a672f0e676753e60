"""Python face of the native ``_tensor_reductions_impl`` module of the reference
(dpnp/tensor/libtensor/source/tensor_reductions.cpp:40-43; sum.cpp:441-456,
max.cpp:401-403, argmax.cpp:270-272): ``_<op>_over_axis(src, trailing_dims_to_reduce,
dst, sycl_queue, depends=[])`` and ``_<op>_over_axis_dtype_supported``.
"""

from __future__ import annotations

import ctypes as C
import sys

from .. import _lib
from .._lib import REDUCE_OPS, SEARCH_OPS, check, lib
from ._tensor_impl import _check_queue, _events, _stream


_nat = _lib.native


def _make_reduce(name, op):
    def call(src, trailing_dims_to_reduce, dst, sycl_queue, depends=()):
        _check_queue(sycl_queue, src, dst)
        if _nat is not None:
            _nat.reduce(op, src._core(), int(trailing_dims_to_reduce), dst._core(), sycl_queue._stream)
            return _events(sycl_queue)
        ds, ks = src._descriptor()
        dd, kd = dst._descriptor()
        check(lib.dpb_reduction_over_axis(op, C.byref(ds), int(trailing_dims_to_reduce), C.byref(dd),
                                          _stream(sycl_queue)))
        return _events(sycl_queue)

    cache = {}

    def supported(arg_dtype, out_dtype, dst_usm_type=None, sycl_queue=None):
        try:
            return cache[(arg_dtype, out_dtype)]
        except (KeyError, TypeError):
            pass
        try:
            ok = bool(lib.dpb_reduce_dtype_supported(op, _lib.typenum_of(arg_dtype),
                                                     _lib.typenum_of(out_dtype)))
        except TypeError:
            return False
        try:
            cache[(arg_dtype, out_dtype)] = ok
        except TypeError:
            pass
        return ok

    call.__name__ = f"_{name}_over_axis"
    supported.__name__ = f"_{name}_over_axis_dtype_supported"
    return call, supported


def _make_search(name, op):
    def call(src, trailing_dims_to_reduce, dst, sycl_queue, depends=()):
        _check_queue(sycl_queue, src, dst)
        if _nat is not None:
            _nat.search(op, src._core(), int(trailing_dims_to_reduce), dst._core(), sycl_queue._stream)
            return _events(sycl_queue)
        ds, ks = src._descriptor()
        dd, kd = dst._descriptor()
        check(lib.dpb_search_over_axis(op, C.byref(ds), int(trailing_dims_to_reduce), C.byref(dd),
                                       _stream(sycl_queue)))
        return _events(sycl_queue)

    call.__name__ = f"_{name}_over_axis"
    return call


_mod = sys.modules[__name__]
for _n, _op in REDUCE_OPS.items():
    _c, _s = _make_reduce(_n, _op)
    setattr(_mod, f"_{_n}_over_axis", _c)
    setattr(_mod, f"_{_n}_over_axis_dtype_supported", _s)
for _n, _op in SEARCH_OPS.items():
    setattr(_mod, f"_{_n}_over_axis", _make_search(_n, _op))
