"""dpnp_b200: the data-parallel core of dpnp (strided elementwise engine and
reduction-over-axis engine) on NVIDIA B200, behind the dpnp Python API.

``import dpnp_b200 as np`` gives the subset of the dpnp namespace that the
elementwise and reduction paths need: ``ndarray``, creation and view functions,
the ufunc objects (add, subtract, multiply, divide, negative, exp, log, sqrt,
erf, comparisons, ...), ``where``, and the reductions sum, prod, mean, max, min,
argmax, argmin, plus ``fuse`` (a chain of elementwise calls as one launch).  All compute runs in hand-written CUDA kernels of
``libdpnp_b200.so``; there is no CPU fallback.
"""

import numpy as _np

from . import _lib, memory, random, scipy, tensor
from ._iface import (all, amax, amin, any, arange, are_same_logical_tensors, argmax, argmin, array, asarray, ascontiguousarray,
                     asnumpy, astype, broadcast_to, check_limitations, copy, copyto, count_nonzero,
                     cumlogsumexp, cumprod, cumsum, cumulative_prod, cumulative_sum,
                     default_float_type, empty, empty_like, expand_dims, flip, from_dlpack, full, full_like,
                     get_result_array, get_usm_ndarray, get_usm_ndarray_or_scalar,
                     is_supported_array_type, linspace, logsumexp, max, mean, min, ones, ones_like, prod, ravel, reduce_hypot, reshape,
                     squeeze, std, sum, transpose, var, where, zeros, zeros_like)
from ._fusion import fuse
from ._ufuncs import (DPNPBinaryFunc, DPNPUnaryFunc, abs, absolute, add, ceil, cos, divide, equal, erf,
                      exp, expm1, floor, greater, greater_equal, isfinite, isinf, isnan, less,
                      less_equal, log, log1p, logical_and, logical_not, logical_or, maximum, minimum,
                      multiply, negative, not_equal, positive, power, reciprocal, sign, sin, sqrt,
                      square, subtract, tanh, true_divide)
from ._ufuncs import (acos, acosh, angle, arccos, arccosh, arcsin, arcsinh, arctan, arctan2, arctanh, asin,
                      asinh, atan, atan2, atanh, bitwise_and, bitwise_invert, bitwise_left_shift,
                      bitwise_not, bitwise_or, bitwise_right_shift, bitwise_xor, cbrt, conj, conjugate,
                      copysign, cosh, exp2, fix, floor_divide, hypot, imag, invert, left_shift, log2,
                      log10, logaddexp, logical_xor, mod, nextafter, proj, real, remainder, right_shift,
                      rint, round, around, rsqrt, signbit, sinh, tan, trunc)
from .dpnp_array import dpnp_array
from .dpnp_array import dpnp_array as ndarray
from .memory import ExecutionPlacementError, StreamQueue, get_default_queue
from . import sharded

__version__ = "0.1.0"

# data types (dpnp/__init__.py:78-116)
bool = bool_ = _np.bool_
int8, int16, int32, int64 = _np.int8, _np.int16, _np.int32, _np.int64
uint8, uint16, uint32, uint64 = _np.uint8, _np.uint16, _np.uint32, _np.uint64
float16, float32, float64 = _np.float16, _np.float32, _np.float64
complex64, complex128 = _np.complex64, _np.complex128
intp = _np.intp
dtype = _np.dtype
finfo, iinfo = _np.finfo, _np.iinfo
nan, inf, pi, e, newaxis = _np.nan, _np.inf, _np.pi, _np.e, None


def isscalar(x):
    return _np.isscalar(x)
