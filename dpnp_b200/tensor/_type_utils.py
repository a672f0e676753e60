"""Type promotion rules of the elementwise and reduction layers.

Restates dpnp/tensor/_type_utils.py: the canonical search order of buffer types
(:37-76), the safe-cast test (:157-177), the search for cast buffers of unary,
binary and in-place operations (:197-266), acceptance rules of divide/negative/
subtract (:89-154), NEP-50 "weak" Python scalars (:312-485) and the default
accumulation types of reductions (:932-972).  A B200 supports both fp16 and
fp64, so no device-dependent relaxations apply.
"""

from __future__ import annotations

import numpy as np

from .._lib import supported_dtypes

_ALL = supported_dtypes()  # bool, i1, u1, ..., f2, f4, f8, c8, c16 in canonical order

DEFAULT_INT = np.dtype("i8")
DEFAULT_UINT = np.dtype("u8")
DEFAULT_FP = np.dtype("f8")
DEFAULT_COMPLEX = np.dtype("c16")
DEFAULT_INDEX = np.dtype("i8")


def _all_data_types():
    return list(_ALL)


def _can_cast(from_, to_, casting="safe"):
    return np.can_cast(from_, to_, casting=casting)


def _get_device_default_dtype(kind):
    return {"b": np.dtype("?"), "i": DEFAULT_INT, "u": DEFAULT_UINT, "f": DEFAULT_FP,
            "c": DEFAULT_COMPLEX}[kind]


# ------------------------------------------------------------ acceptance rules
def _acceptance_fn_default_unary(arg_dtype, buf_dt, res_dt):
    return True


def _acceptance_fn_default_binary(arg1_dtype, arg2_dtype, buf1_dt, buf2_dt, res_dt):
    return True


def _acceptance_fn_divide(arg1_dtype, arg2_dtype, buf1_dt, buf2_dt, res_dt):
    # when both operands change kind (e.g. int8 / uint8) the result must be the
    # default type of the resulting kind, as in NumPy, not the smallest float
    if buf1_dt.kind != arg1_dtype.kind and buf2_dt.kind != arg2_dtype.kind:
        return res_dt == _get_device_default_dtype(res_dt.kind)
    return True


def _acceptance_fn_negative(arg_dtype, buf_dt, res_dt):
    if arg_dtype.char == "?":
        raise ValueError(
            "The `negative` function, the `-` operator, is not supported for inputs of data type "
            "bool, use the `~` operator or the `logical_not` function instead")
    return True


def _acceptance_fn_reciprocal(arg_dtype, buf_dt, res_dt):
    """When the input must change kind (an integer array), only the default floating type of
    the result kind is accepted, which keeps reciprocal and divide aligned
    (dpnp/tensor/_type_utils.py:122-133)."""
    if buf_dt.kind != arg_dtype.kind:
        return res_dt == _get_device_default_dtype(res_dt.kind)
    return True


def _acceptance_fn_round(arg_dtype, buf_dt, res_dt):
    """Boolean input rounds to a floating result, not an integral one
    (dpnp/tensor/_type_utils.py:136-140)."""
    return not (arg_dtype.kind == "b" and res_dt.kind != "f")


def _acceptance_fn_subtract(arg1_dtype, arg2_dtype, buf1_dt, buf2_dt, res_dt):
    if arg1_dtype.char == "?" and arg2_dtype.char == "?":
        raise ValueError(
            "The `subtract` function, the `-` operator, is not supported for inputs of data type "
            "bool, use the `^` operator,  the `bitwise_xor`, or the `logical_xor` function instead")
    return True


# ------------------------------------------------------------- buffer search
def _find_buf_dtype(arg_dtype, query_fn, acceptance_fn=_acceptance_fn_default_unary):
    """(buffer dtype or None, result dtype or None) for a unary operation."""
    res = query_fn(arg_dtype)
    if res:
        return None, res
    for buf in _ALL:
        if _can_cast(arg_dtype, buf):
            res = query_fn(buf)
            if res and acceptance_fn(arg_dtype, buf, res):
                return buf, res
    return None, None


def _find_buf_dtype2(arg1_dtype, arg2_dtype, query_fn, acceptance_fn=_acceptance_fn_default_binary):
    """(buffer1, buffer2, result) for a binary operation; a buffer of None means no cast."""
    res = query_fn(arg1_dtype, arg2_dtype)
    if res:
        return None, None, res
    for buf1 in _ALL:
        if not _can_cast(arg1_dtype, buf1):
            continue
        for buf2 in _ALL:
            if not _can_cast(arg2_dtype, buf2):
                continue
            res = query_fn(buf1, buf2)
            if not res:
                continue
            r1 = None if buf1 == arg1_dtype else buf1
            r2 = None if buf2 == arg2_dtype else buf2
            if r1 is None or r2 is None:
                return r1, r2, res
            if acceptance_fn(arg1_dtype, arg2_dtype, r1, r2, res):
                return r1, r2, res
    return None, None, None


def _find_buf_dtype_in_place_op(arg1_dtype, arg2_dtype, query_fn):
    res = query_fn(arg1_dtype, arg2_dtype)
    if res:
        return None, res
    if _can_cast(arg2_dtype, arg1_dtype, casting="same_kind"):
        res = query_fn(arg1_dtype, arg1_dtype)
        if res:
            return arg1_dtype, res
    return None, None


# ----------------------------------------------------------------- weak types
class _Weak:
    kind_num = -1

    def __init__(self, o):
        self.o_ = o

    def get(self):
        return self.o_


class WeakBooleanType(_Weak):
    kind_num = 0


class WeakIntegralType(_Weak):
    kind_num = 1


class WeakFloatingType(_Weak):
    kind_num = 2


class WeakComplexType(_Weak):
    kind_num = 3


def _is_weak_dtype(dt):
    return isinstance(dt, _Weak)


_KIND_NUM = {"b": 0, "i": 1, "u": 1, "f": 2, "c": 3}


def _promote_weak(weak, strong, check_int_range):
    """dtype standing for a weak scalar next to a strong dtype."""
    wk, sk = weak.kind_num, _KIND_NUM[strong.kind]
    if wk > sk:
        if isinstance(weak, WeakIntegralType):
            return DEFAULT_INT
        if isinstance(weak, WeakComplexType):
            return np.dtype("c8") if strong in (np.dtype("f2"), np.dtype("f4")) else DEFAULT_COMPLEX
        return DEFAULT_FP
    if check_int_range and wk == sk and isinstance(weak, WeakIntegralType):
        v = weak.get()
        info = np.iinfo(strong)
        if v < info.min or v > info.max:
            return np.dtype(np.min_scalar_type(v))
    return strong


def _resolve_weak_types(o1_dtype, o2_dtype, dev=None):
    """NEP-50 resolution when at most one operand is a Python scalar."""
    if _is_weak_dtype(o1_dtype):
        if _is_weak_dtype(o2_dtype):
            raise ValueError
        return _promote_weak(o1_dtype, o2_dtype, False), o2_dtype
    if _is_weak_dtype(o2_dtype):
        return o1_dtype, _promote_weak(o2_dtype, o1_dtype, False)
    return o1_dtype, o2_dtype


def _resolve_weak_types_all_py_ints(o1_dtype, o2_dtype, dev=None):
    """Variant for comparisons and divide: a Python int outside the range of the
    array's integer type keeps its own minimal type instead of overflowing."""
    if _is_weak_dtype(o1_dtype):
        if _is_weak_dtype(o2_dtype):
            raise ValueError
        return _promote_weak(o1_dtype, o2_dtype, True), o2_dtype
    if _is_weak_dtype(o2_dtype):
        return o1_dtype, _promote_weak(o2_dtype, o1_dtype, True)
    return o1_dtype, o2_dtype


def _resolve_one_strong_two_weak_types(st_dtype, dtype1, dtype2, dev=None):
    """`where(cond, x1, x2)` with Python scalars for x1 and/or x2."""
    if _is_weak_dtype(st_dtype):
        raise ValueError
    if _is_weak_dtype(dtype1) and _is_weak_dtype(dtype2):
        k = max(dtype1.kind_num, dtype2.kind_num)
        sk = _KIND_NUM[st_dtype.kind]
        if k > sk:
            dt = {1: DEFAULT_INT, 2: DEFAULT_FP, 3: DEFAULT_COMPLEX}[k]
            return dt, dt
        return st_dtype, st_dtype
    if _is_weak_dtype(dtype1):
        d1 = _promote_weak(dtype1, np.result_type(st_dtype, dtype2), False)
        return d1, dtype2
    if _is_weak_dtype(dtype2):
        d2 = _promote_weak(dtype2, np.result_type(st_dtype, dtype1), False)
        return dtype1, d2
    return dtype1, dtype2


def _get_dtype(o):
    """dtype of an operand; Python scalars map to weak types."""
    if hasattr(o, "dtype") and hasattr(o, "shape"):
        return np.dtype(o.dtype)
    if isinstance(o, (bool, np.bool_)):
        return WeakBooleanType(o) if isinstance(o, bool) else np.dtype("?")
    if isinstance(o, np.generic):
        return o.dtype
    if isinstance(o, int):
        return WeakIntegralType(o)
    if isinstance(o, float):
        return WeakFloatingType(o)
    if isinstance(o, complex):
        return WeakComplexType(o)
    return np.dtype(object)


def _validate_dtype(dt):
    return _is_weak_dtype(dt) or dt in _ALL


def _get_shape(o):
    if hasattr(o, "shape"):
        return tuple(o.shape)
    if isinstance(o, (bool, int, float, complex, np.generic)):
        return ()
    return getattr(o, "shape", None)


# ---------------------------------------------------------------- reductions
def _default_accumulation_dtype(inp_dt):
    """Result type of sum/prod when none is given: bool and signed integers
    accumulate in int64, unsigned in uint64, floating and complex keep their type."""
    k = inp_dt.kind
    if k in "bi":
        return DEFAULT_INT if np.can_cast(inp_dt, DEFAULT_INT) else inp_dt
    if k == "u":
        return DEFAULT_UINT if np.can_cast(inp_dt, DEFAULT_UINT) else inp_dt
    return inp_dt


def _default_accumulation_dtype_fp_types(inp_dt):
    """Result type of floating-only accumulations (mean, logsumexp): non-floating
    inputs use the default floating type."""
    if inp_dt.kind in "biu":
        return DEFAULT_FP
    return inp_dt


def result_type(*arrays_and_dtypes):
    """Array-API result_type over arrays, dtypes and Python scalars."""
    strong = []
    weak = []
    for a in arrays_and_dtypes:
        if isinstance(a, (bool, int, float, complex)) and not isinstance(a, np.generic):
            weak.append(a)
        elif hasattr(a, "dtype") and hasattr(a, "shape"):
            strong.append(np.dtype(a.dtype))
        else:
            strong.append(np.dtype(a))
    if not strong:
        return np.result_type(*weak)
    res = np.result_type(*strong)
    for w in weak:
        res = _promote_weak(_get_dtype(w), res, False) if _is_weak_dtype(_get_dtype(w)) else res
    return res


def can_cast(from_, to, /, *, casting="safe"):
    f = from_.dtype if hasattr(from_, "dtype") else np.dtype(from_)
    return np.can_cast(f, np.dtype(to), casting=casting)
