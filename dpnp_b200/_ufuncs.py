"""NumPy-style ufunc objects of the public API.

``DPNPUnaryFunc`` / ``DPNPBinaryFunc`` add the NumPy keyword handling of the
reference classes (dpnp/dpnp_algo/dpnp_elementwise_common.py:81-235,537-739) on
top of the tensor-level function objects: ``out`` (array or 1-tuple), ``where``
and ``subok`` must keep their defaults, ``dtype`` casts the inputs first and
excludes ``out``, ``x1 is out`` takes the in-place kernel.  There is no
vendor-library fast path: every call runs the library's own kernels.
"""

from __future__ import annotations

import numpy as np

from . import _fusion
from . import tensor as dpt
from .dpnp_array import dpnp_array
from .sharded import ShardedArray
from .sharded import elementwise as _sharded_elementwise
from .tensor import _elementwise_funcs as ef
from .tensor._elementwise_common import BinaryElementwiseFunc, UnaryElementwiseFunc
from .tensor._usmarray import usm_ndarray


def _is_array(x):
    return isinstance(x, (dpnp_array, usm_ndarray))


def _is_scalar(x):
    return isinstance(x, (bool, int, float, complex, np.generic))


def _usm(x):
    return x._array_obj if isinstance(x, dpnp_array) else x


def _check_common_kwargs(name, kwargs, where, subok, dtype, out):
    if kwargs:
        raise NotImplementedError(f"Requested function={name} with kwargs={kwargs} isn't currently supported.")
    if where is not True:
        raise NotImplementedError(f"Requested function={name} with where={where} isn't currently supported.")
    if subok is not True:
        raise NotImplementedError(f"Requested function={name} with subok={subok} isn't currently supported.")
    if dtype is not None and out is not None:
        raise TypeError(f"Requested function={name} only takes `out` or `dtype` as an argument, "
                        "but both were provided.")


def _norm_order(order):
    if order is None:
        return "K"
    if isinstance(order, str) and order in "afkcAFKC" and len(order) == 1:
        return order.upper()
    raise ValueError(f"order must be one of 'C', 'F', 'A', or 'K' (got '{order}')")


def _wrap_new(usm_ary):
    res = dpnp_array.__new__(dpnp_array)
    res._array_obj = usm_ary
    return res


def _unpack_out(out, nout=1):
    if isinstance(out, tuple):
        if len(out) != nout:
            raise ValueError("'out' tuple must have exactly one entry per ufunc output")
        return out[0]
    return out


class DPNPUnaryFunc(UnaryElementwiseFunc):
    def __init__(self, base: UnaryElementwiseFunc, name=None, docs=None):
        super().__init__(name or base.name_, base.result_type_resolver_fn_, base.unary_fn_,
                         docs or base.__doc__, acceptance_fn=base.acceptance_fn_)
        self.__name__ = "DPNPUnaryFunc"

    def __call__(self, x, /, out=None, *, where=True, order="K", dtype=None, subok=True, **kwargs):
        if (type(x) is dpnp_array and out is None and dtype is None and order == "K" and where is True
                and subok is True and not kwargs):
            # the plain call f(x): nothing to check beyond what the tensor-level object checks
            return _wrap_new(UnaryElementwiseFunc.__call__(self, x._array_obj))
        if type(x) is ShardedArray:                # slab-wise on every rank, no communication
            _check_common_kwargs(self.name_, kwargs, where, subok, dtype, out)
            kw = {k: v for k, v in (("out", out), ("dtype", dtype)) if v is not None}
            return _sharded_elementwise(self._public_name, x, order=order, **kw)
        _check_common_kwargs(self.name_, kwargs, where, subok, dtype, out)
        if type(x) is _fusion.FusedValue:          # inside a function that is being fused
            if dtype is not None:
                raise _fusion.FusionUnsupported("dtype= inside a fused function")
            return _fusion.trace_unary(self.name_, x, out)
        if not _is_array(x):
            raise TypeError(f"Input array must be any of supported type, but got {type(x)}")
        order = _norm_order(order)
        x_usm = _usm(x)
        if dtype is not None:
            x_usm = dpt.astype(x_usm, dtype, copy=False)
        out = _unpack_out(out)
        if out is not None and not _is_array(out):
            raise TypeError(f"output array must be any of supported type, but got {type(out)}")
        res = super().__call__(x_usm, out=None if out is None else _usm(out), order=order)
        if out is not None and isinstance(out, dpnp_array):
            return out
        return dpnp_array._create_from_usm_ndarray(res)


class DPNPBinaryFunc(BinaryElementwiseFunc):
    def __init__(self, base: BinaryElementwiseFunc, name=None, docs=None):
        super().__init__(name or base.name_, base.result_type_resolver_fn_, base.binary_fn_,
                         docs or base.__doc__, binary_inplace_fn=base.binary_inplace_fn_,
                         acceptance_fn=base.acceptance_fn_, weak_type_resolver=base.weak_type_resolver_)
        self.__name__ = "DPNPBinaryFunc"

    def __call__(self, x1, x2, /, out=None, *, where=True, order="K", dtype=None, subok=True, **kwargs):
        if (out is None and dtype is None and order == "K" and where is True and subok is True
                and not kwargs):
            # the plain call f(x1, x2) on arrays, or an array and a Python float/int
            t1, t2 = type(x1), type(x2)
            if t1 is dpnp_array:
                if t2 is dpnp_array:
                    return _wrap_new(BinaryElementwiseFunc.__call__(self, x1._array_obj, x2._array_obj))
                if t2 is float or t2 is int:
                    return _wrap_new(BinaryElementwiseFunc.__call__(self, x1._array_obj, x2))
            elif t2 is dpnp_array and (t1 is float or t1 is int):
                return _wrap_new(BinaryElementwiseFunc.__call__(self, x1, x2._array_obj))
        if type(x1) is ShardedArray or type(x2) is ShardedArray:
            _check_common_kwargs(self.name_, kwargs, where, subok, dtype, out)
            kw = {k: v for k, v in (("out", out), ("dtype", dtype)) if v is not None}
            return _sharded_elementwise(self._public_name, x1, x2, order=order, **kw)
        if _fusion.is_traced(x1, x2):              # inside a function that is being fused
            _check_common_kwargs(self.name_, kwargs, where, subok, dtype, out)
            if dtype is not None:
                raise _fusion.FusionUnsupported("dtype= inside a fused function")
            return _fusion.trace_binary(self.name_, x1, x2, out)
        t1, t2 = type(x1), type(x2)
        if not (t1 is dpnp_array and t2 is dpnp_array):
            for x in (x1, x2):
                if not (_is_array(x) or _is_scalar(x)):
                    raise TypeError(f"An array must be any of supported type, but got {type(x)}")
            if not (_is_array(x1) or _is_array(x2)):
                raise TypeError("Input should be any of supported array type, got two scalars")
        if kwargs or where is not True or subok is not True or (dtype is not None and out is not None):
            _check_common_kwargs(self.name_, kwargs, where, subok, dtype, out)
        x1_usm, x2_usm = _usm(x1), _usm(x2)
        out = _unpack_out(out)
        if out is not None and not _is_array(out):
            raise TypeError(f"output array must be any of supported type, but got {type(out)}")
        out_usm = None if out is None else _usm(out)
        if isinstance(x1, dpnp_array) and x1 is out and order == "K" and dtype is None:
            super()._inplace_op(x1_usm, x2_usm)
            return x1
        order = _norm_order(order)
        if dtype is not None:
            if _is_scalar(x1):
                x1_usm = dpt.asarray(x1, dtype=dtype, sycl_queue=x2_usm.sycl_queue)
                x2_usm = dpt.astype(x2_usm, dtype, copy=False)
            elif _is_scalar(x2):
                x1_usm = dpt.astype(x1_usm, dtype, copy=False)
                x2_usm = dpt.asarray(x2, dtype=dtype, sycl_queue=x1_usm.sycl_queue)
            else:
                x1_usm = dpt.astype(x1_usm, dtype, copy=False)
                x2_usm = dpt.astype(x2_usm, dtype, copy=False)
        res = super().__call__(x1_usm, x2_usm, out=out_usm, order=order)
        if out is not None and isinstance(out, dpnp_array):
            return out
        return dpnp_array._create_from_usm_ndarray(res)


# unary
abs = absolute = DPNPUnaryFunc(ef.abs, "abs")
negative = DPNPUnaryFunc(ef.negative)
positive = DPNPUnaryFunc(ef.positive)
exp = DPNPUnaryFunc(ef.exp)
log = DPNPUnaryFunc(ef.log)
sqrt = DPNPUnaryFunc(ef.sqrt)
erf = DPNPUnaryFunc(ef.erf)
square = DPNPUnaryFunc(ef.square)
reciprocal = DPNPUnaryFunc(ef.reciprocal)
sin = DPNPUnaryFunc(ef.sin)
cos = DPNPUnaryFunc(ef.cos)
tanh = DPNPUnaryFunc(ef.tanh)
expm1 = DPNPUnaryFunc(ef.expm1)
log1p = DPNPUnaryFunc(ef.log1p)
floor = DPNPUnaryFunc(ef.floor)
ceil = DPNPUnaryFunc(ef.ceil)
sign = DPNPUnaryFunc(ef.sign)
logical_not = DPNPUnaryFunc(ef.logical_not)
isnan = DPNPUnaryFunc(ef.isnan)
isfinite = DPNPUnaryFunc(ef.isfinite)
isinf = DPNPUnaryFunc(ef.isinf)
# binary
add = DPNPBinaryFunc(ef.add)
subtract = DPNPBinaryFunc(ef.subtract)
multiply = DPNPBinaryFunc(ef.multiply)
divide = true_divide = DPNPBinaryFunc(ef.divide, "divide")
maximum = DPNPBinaryFunc(ef.maximum)
minimum = DPNPBinaryFunc(ef.minimum)
power = DPNPBinaryFunc(ef.pow, "power")
equal = DPNPBinaryFunc(ef.equal)
not_equal = DPNPBinaryFunc(ef.not_equal)
less = DPNPBinaryFunc(ef.less)
less_equal = DPNPBinaryFunc(ef.less_equal)
greater = DPNPBinaryFunc(ef.greater)
greater_equal = DPNPBinaryFunc(ef.greater_equal)
logical_and = DPNPBinaryFunc(ef.logical_and)
logical_or = DPNPBinaryFunc(ef.logical_or)

# the rest of the elementwise family, NumPy names (dpnp/dpnp_iface_trigonometric.py,
# dpnp_iface_mathematical.py, dpnp_iface_bitwise.py, dpnp_iface_logic.py)
acos = arccos = DPNPUnaryFunc(ef.acos, "acos")
acosh = arccosh = DPNPUnaryFunc(ef.acosh, "acosh")
asin = arcsin = DPNPUnaryFunc(ef.asin, "asin")
asinh = arcsinh = DPNPUnaryFunc(ef.asinh, "asinh")
atan = arctan = DPNPUnaryFunc(ef.atan, "atan")
atanh = arctanh = DPNPUnaryFunc(ef.atanh, "atanh")
cbrt = DPNPUnaryFunc(ef.cbrt)
cosh = DPNPUnaryFunc(ef.cosh)
sinh = DPNPUnaryFunc(ef.sinh)
tan = DPNPUnaryFunc(ef.tan)
exp2 = DPNPUnaryFunc(ef.exp2)
log2 = DPNPUnaryFunc(ef.log2)
log10 = DPNPUnaryFunc(ef.log10)
rsqrt = DPNPUnaryFunc(ef.rsqrt)
trunc = fix = DPNPUnaryFunc(ef.trunc)
rint = DPNPUnaryFunc(ef.round, "rint")
signbit = DPNPUnaryFunc(ef.signbit)
invert = bitwise_not = bitwise_invert = DPNPUnaryFunc(ef.bitwise_invert, "invert")
conj = conjugate = DPNPUnaryFunc(ef.conj, "conjugate")
real = DPNPUnaryFunc(ef.real)
imag = DPNPUnaryFunc(ef.imag)
angle = DPNPUnaryFunc(ef.angle)
proj = DPNPUnaryFunc(ef.proj)
atan2 = arctan2 = DPNPBinaryFunc(ef.atan2, "atan2")
hypot = DPNPBinaryFunc(ef.hypot)
copysign = DPNPBinaryFunc(ef.copysign)
logaddexp = DPNPBinaryFunc(ef.logaddexp)
nextafter = DPNPBinaryFunc(ef.nextafter)
bitwise_and = DPNPBinaryFunc(ef.bitwise_and)
bitwise_or = DPNPBinaryFunc(ef.bitwise_or)
bitwise_xor = DPNPBinaryFunc(ef.bitwise_xor)
left_shift = bitwise_left_shift = DPNPBinaryFunc(ef.bitwise_left_shift, "left_shift")
right_shift = bitwise_right_shift = DPNPBinaryFunc(ef.bitwise_right_shift, "right_shift")
floor_divide = DPNPBinaryFunc(ef.floor_divide)
remainder = mod = DPNPBinaryFunc(ef.remainder)
logical_xor = DPNPBinaryFunc(ef.logical_xor)


class DPNPRound(DPNPUnaryFunc):
    """dpnp.round / dpnp.around: rounding to `decimals` places by scaling, rounding half to even
    and scaling back (dpnp/dpnp_algo/dpnp_elementwise_common.py:1290-1341)."""

    def __call__(self, x, /, decimals=0, out=None, *, dtype=None):
        if decimals == 0:
            return super().__call__(x, out=out, dtype=dtype)
        x_usm = _usm(x)
        out = _unpack_out(out)
        out_usm = None if out is None else _usm(out)
        if x_usm.dtype.kind in "iu":
            if decimals < 0:
                dtype = x_usm.dtype
                x_usm = ef.round(x_usm * 10 ** decimals, out=out_usm)
                res_usm = ef.divide(x_usm, 10 ** decimals, out=out_usm)
            else:
                res_usm = ef.round(x_usm, out=out_usm)
        else:
            x_usm = ef.round(x_usm * 10 ** decimals, out=out_usm)
            res_usm = ef.divide(x_usm, 10 ** decimals, out=out_usm)
        if dtype is not None:
            res_usm = dpt.astype(res_usm, dtype, copy=False)
        if out is not None and isinstance(out, dpnp_array):
            return out
        return dpnp_array._create_from_usm_ndarray(res_usm)


round = around = DPNPRound(ef.round, "round")


# name under which each ufunc object is reachable in the package (and in NumPy): sharded arrays
# apply the function of that name to their local parts
for _n, _o in list(globals().items()):
    if isinstance(_o, (DPNPUnaryFunc, DPNPBinaryFunc)) and not hasattr(_o, "_public_name"):
        _o._public_name = _n
