"""Python face of the native ``_tensor_accumulation_impl`` module of the reference
(dpnp/tensor/libtensor/source/tensor_accumulation.cpp; cumulative_sum.cpp, cumulative_prod.cpp,
cumulative_logsumexp.cpp): ``_<op>_over_axis(src, trailing_dims_to_accumulate, dst, sycl_queue)``,
``_<op>_final_axis_include_initial(src, dst, sycl_queue)`` and ``_<op>_dtype_supported``."""

from __future__ import annotations

import ctypes as C
import sys

from .. import _lib
from .._lib import ACCUMULATE_OPS, check, lib
from ._tensor_impl import _check_queue, _events, _stream


def _make(name, op):
    def over_axis(src, trailing_dims_to_accumulate, dst, sycl_queue, depends=()):
        if trailing_dims_to_accumulate != 1:
            raise ValueError("accumulation is carried out over one trailing dimension")
        _check_queue(sycl_queue, src, dst)
        if _lib.native is not None:
            _lib.native.accumulate(op, src._core(), dst._core(), 0, sycl_queue._stream)
            return _events(sycl_queue)
        ds, ks = src._descriptor()
        dd, kd = dst._descriptor()
        check(lib.dpb_accumulate_over_axis(op, C.byref(ds), C.byref(dd), 0, _stream(sycl_queue)))
        return _events(sycl_queue)

    def include_initial(src, dst, sycl_queue, depends=()):
        _check_queue(sycl_queue, src, dst)
        if _lib.native is not None:
            _lib.native.accumulate(op, src._core(), dst._core(), 1, sycl_queue._stream)
            return _events(sycl_queue)
        ds, ks = src._descriptor()
        dd, kd = dst._descriptor()
        check(lib.dpb_accumulate_over_axis(op, C.byref(ds), C.byref(dd), 1, _stream(sycl_queue)))
        return _events(sycl_queue)

    def supported(arg_dtype, out_dtype):
        try:
            return bool(lib.dpb_accumulate_dtype_supported(op, _lib.typenum_of(arg_dtype),
                                                           _lib.typenum_of(out_dtype)))
        except TypeError:
            return False

    over_axis.__name__ = f"_{name}_over_axis"
    include_initial.__name__ = f"_{name}_final_axis_include_initial"
    supported.__name__ = f"_{name}_dtype_supported"
    return over_axis, include_initial, supported


_mod = sys.modules[__name__]
for _n, _op in ACCUMULATE_OPS.items():
    _a, _b, _c = _make(_n, _op)
    setattr(_mod, f"_{_n}_over_axis", _a)
    setattr(_mod, f"_{_n}_final_axis_include_initial", _b)
    setattr(_mod, f"_{_n}_dtype_supported", _c)
