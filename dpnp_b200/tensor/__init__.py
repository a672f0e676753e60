"""Array-API style tensor layer over libdpnp_b200 (the role dpnp.tensor plays in
the reference): the ``usm_ndarray`` object, creation and manipulation functions,
the elementwise function objects, reductions, ``where`` and ``mean``."""

import numpy as _np

from ..memory import ExecutionPlacementError, StreamQueue, get_default_queue
from ._copy_utils import asnumpy, astype, copy, from_numpy, to_numpy
from ._ctors import (arange, asarray, empty, empty_like, full, full_like, linspace, ones, ones_like, zeros,
                     zeros_like)
from ._dlpack import from_dlpack
from ._elementwise_funcs import (abs, add, ceil, cos, divide, equal, erf, exp, expm1, floor, greater,
                                 greater_equal, isfinite, isinf, isnan, less, less_equal, log, log1p,
                                 logical_and, logical_not, logical_or, maximum, minimum, multiply,
                                 negative, not_equal, positive, pow, reciprocal, sign, sin, sqrt,
                                 square, subtract, tanh)
from ._elementwise_funcs import (acos, acosh, angle, asin, asinh, atan, atan2, atanh, bitwise_and,
                                 bitwise_invert, bitwise_left_shift, bitwise_or, bitwise_right_shift,
                                 bitwise_xor, cbrt, conj, copysign, cosh, exp2, floor_divide, hypot, imag,
                                 log2, log10, logaddexp, logical_xor, nextafter, proj, real, remainder,
                                 round, rsqrt, signbit, sinh, tan, trunc)
from ._manipulation_functions import (broadcast_arrays, broadcast_shapes, broadcast_to, expand_dims,
                                      flip, permute_dims, reshape, squeeze)
from ._reduction import (all, any, argmax, argmin, count_nonzero, logsumexp, max, min, prod, reduce_hypot,
                         sum)
from ._search_functions import where
from ._accumulation import cumulative_logsumexp, cumulative_prod, cumulative_sum
from ._statistical_functions import mean, std, var
from ._type_utils import can_cast, result_type
from ._usmarray import usm_ndarray

dtype = _np.dtype
bool = _np.dtype("?")
int8 = _np.dtype("i1")
uint8 = _np.dtype("u1")
int16 = _np.dtype("i2")
uint16 = _np.dtype("u2")
int32 = _np.dtype("i4")
uint32 = _np.dtype("u4")
int64 = _np.dtype("i8")
uint64 = _np.dtype("u8")
float16 = _np.dtype("f2")
float32 = _np.dtype("f4")
float64 = _np.dtype("f8")
complex64 = _np.dtype("c8")
complex128 = _np.dtype("c16")
