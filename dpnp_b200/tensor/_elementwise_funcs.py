"""The elementwise function objects (dpnp/tensor/_elementwise_funcs.py of the
reference defines the same names the same way: one ``UnaryElementwiseFunc`` or
``BinaryElementwiseFunc`` per operation, bound to its native implementation,
result-type query and, where the reference has them, acceptance rule and weak
type resolver)."""

from __future__ import annotations

from . import _tensor_elementwise_impl as tei
from ._elementwise_common import BinaryElementwiseFunc, UnaryElementwiseFunc
from ._type_utils import (_acceptance_fn_divide, _acceptance_fn_negative, _acceptance_fn_reciprocal,
                          _acceptance_fn_round, _acceptance_fn_subtract, _resolve_weak_types_all_py_ints)


def _unary(name, doc, **kw):
    return UnaryElementwiseFunc(name, getattr(tei, f"_{name}_result_type"), getattr(tei, f"_{name}"),
                                doc, **kw)


def _binary(name, doc, inplace=True, **kw):
    return BinaryElementwiseFunc(
        name, getattr(tei, f"_{name}_result_type"), getattr(tei, f"_{name}"), doc,
        binary_inplace_fn=getattr(tei, f"_{name}_inplace") if inplace else None, **kw)


abs = _unary("abs", "abs(x, /, *, out=None, order='K'): absolute value of each element.")
negative = _unary("negative", "negative(x, /, *, out=None, order='K'): numerical negative of each element.",
                  acceptance_fn=_acceptance_fn_negative)
positive = _unary("positive", "positive(x, /, *, out=None, order='K'): numerical positive of each element.")
exp = _unary("exp", "exp(x, /, *, out=None, order='K'): exponential of each element.")
log = _unary("log", "log(x, /, *, out=None, order='K'): natural logarithm of each element.")
sqrt = _unary("sqrt", "sqrt(x, /, *, out=None, order='K'): square root of each element.")
erf = _unary("erf", "erf(x, /, *, out=None, order='K'): error function of each element.")
square = _unary("square", "square(x, /, *, out=None, order='K'): square of each element.")
reciprocal = _unary("reciprocal", "reciprocal(x, /, *, out=None, order='K'): 1/x for each element.",
                    acceptance_fn=_acceptance_fn_reciprocal)
sin = _unary("sin", "sin(x, /, *, out=None, order='K'): sine of each element.")
cos = _unary("cos", "cos(x, /, *, out=None, order='K'): cosine of each element.")
tanh = _unary("tanh", "tanh(x, /, *, out=None, order='K'): hyperbolic tangent of each element.")
expm1 = _unary("expm1", "expm1(x, /, *, out=None, order='K'): exp(x)-1 for each element.")
log1p = _unary("log1p", "log1p(x, /, *, out=None, order='K'): log(1+x) for each element.")
floor = _unary("floor", "floor(x, /, *, out=None, order='K'): floor of each element.")
ceil = _unary("ceil", "ceil(x, /, *, out=None, order='K'): ceiling of each element.")
sign = _unary("sign", "sign(x, /, *, out=None, order='K'): sign of each element.")
logical_not = _unary("logical_not", "logical_not(x, /, *, out=None, order='K'): logical NOT of each element.")
isnan = _unary("isnan", "isnan(x, /, *, out=None, order='K'): test each element for NaN.")
isfinite = _unary("isfinite", "isfinite(x, /, *, out=None, order='K'): test each element for finiteness.")
isinf = _unary("isinf", "isinf(x, /, *, out=None, order='K'): test each element for infinity.")

add = _binary("add", "add(x1, x2, /, *, out=None, order='K'): elementwise sum.")
subtract = _binary("subtract", "subtract(x1, x2, /, *, out=None, order='K'): elementwise difference.",
                   acceptance_fn=_acceptance_fn_subtract)
multiply = _binary("multiply", "multiply(x1, x2, /, *, out=None, order='K'): elementwise product.")
divide = _binary("divide", "divide(x1, x2, /, *, out=None, order='K'): elementwise true division.",
                 acceptance_fn=_acceptance_fn_divide, weak_type_resolver=_resolve_weak_types_all_py_ints)
maximum = _binary("maximum", "maximum(x1, x2, /, *, out=None, order='K'): elementwise maximum (NaN propagates).")
minimum = _binary("minimum", "minimum(x1, x2, /, *, out=None, order='K'): elementwise minimum (NaN propagates).")
pow = _binary("pow", "pow(x1, x2, /, *, out=None, order='K'): x1 raised to the power x2.")
equal = _binary("equal", "equal(x1, x2, /, *, out=None, order='K'): x1 == x2.", inplace=False,
                weak_type_resolver=_resolve_weak_types_all_py_ints)
not_equal = _binary("not_equal", "not_equal(x1, x2, /, *, out=None, order='K'): x1 != x2.", inplace=False,
                    weak_type_resolver=_resolve_weak_types_all_py_ints)
less = _binary("less", "less(x1, x2, /, *, out=None, order='K'): x1 < x2.", inplace=False,
               weak_type_resolver=_resolve_weak_types_all_py_ints)
less_equal = _binary("less_equal", "less_equal(x1, x2, /, *, out=None, order='K'): x1 <= x2.", inplace=False,
                     weak_type_resolver=_resolve_weak_types_all_py_ints)
greater = _binary("greater", "greater(x1, x2, /, *, out=None, order='K'): x1 > x2.", inplace=False,
                  weak_type_resolver=_resolve_weak_types_all_py_ints)
greater_equal = _binary("greater_equal", "greater_equal(x1, x2, /, *, out=None, order='K'): x1 >= x2.",
                        inplace=False, weak_type_resolver=_resolve_weak_types_all_py_ints)
logical_and = _binary("logical_and", "logical_and(x1, x2, /, *, out=None, order='K'): x1 AND x2.", inplace=False)
logical_or = _binary("logical_or", "logical_or(x1, x2, /, *, out=None, order='K'): x1 OR x2.", inplace=False)

# the rest of the elementwise family (dpnp/tensor/_elementwise_funcs.py defines one object per
# source file under libtensor/source/elementwise_functions/)
_SIG1 = "(x, /, *, out=None, order='K')"
_SIG2 = "(x1, x2, /, *, out=None, order='K')"
for _name, _what in (
        ("acos", "inverse cosine"), ("acosh", "inverse hyperbolic cosine"), ("asin", "inverse sine"),
        ("asinh", "inverse hyperbolic sine"), ("atan", "inverse tangent"),
        ("atanh", "inverse hyperbolic tangent"), ("cbrt", "cube root"), ("cosh", "hyperbolic cosine"),
        ("sinh", "hyperbolic sine"), ("tan", "tangent"), ("exp2", "2**x"), ("log2", "base-2 logarithm"),
        ("log10", "base-10 logarithm"), ("rsqrt", "reciprocal square root"),
        ("trunc", "value rounded towards zero"), ("signbit", "True where the sign bit is set"),
        ("bitwise_invert", "bitwise complement (logical not for bool)"), ("conj", "complex conjugate"),
        ("real", "real part"), ("imag", "imaginary part"), ("angle", "argument of a complex number"),
        ("proj", "projection onto the Riemann sphere")):
    globals()[_name] = _unary(_name, f"{_name}{_SIG1}: {_what} of each element.")
round = _unary("round", f"round{_SIG1}: each element rounded to the nearest integer, halves to even.",
               acceptance_fn=_acceptance_fn_round)
for _name, _what, _inplace in (
        ("atan2", "inverse tangent of x1/x2 in the right quadrant", True),
        ("hypot", "sqrt(x1**2 + x2**2) without undue overflow", True),
        ("copysign", "x1 with the sign of x2", True),
        ("logaddexp", "log(exp(x1) + exp(x2))", True),
        ("nextafter", "next representable value after x1 towards x2", True),
        ("bitwise_and", "bitwise AND", True), ("bitwise_or", "bitwise OR", True),
        ("bitwise_xor", "bitwise XOR", True),
        ("bitwise_left_shift", "x1 shifted left by x2 bits", True),
        ("bitwise_right_shift", "x1 shifted right by x2 bits", True),
        ("floor_divide", "floor of x1 / x2", True), ("remainder", "x1 modulo x2 (sign of x2)", True),
        ("logical_xor", "x1 XOR x2", False)):
    globals()[_name] = _binary(_name, f"{_name}{_SIG2}: {_what}, elementwise.", inplace=_inplace)
del _name, _what, _inplace
