"""TEST INFRASTRUCTURE, not product code: the CPU oracle for the elementwise and
reduction path of dpnp.

Only ``tests/``, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py`` may import this module.  It restates,
with NumPy on the host, what the reference computes for the path, citing the
reference code each function follows (paths relative to the root of
IntelPython/dpnp), and loads two native helpers:

* ``liboracle_core.so`` -- the plain-C restatement in ``oracle_core.c``;
* ``_ref/libref_strided_iters.so`` -- the reference's own iteration-space
  simplifier compiled from its SYCL-free header (``kind: reference`` evidence
  for that one piece of host logic).

Parity status: the reference itself cannot be built or imported in this
environment (DPC++/SYCL, dpctl and oneMKL are absent), so the oracle is pinned
against the known-answer cases of the reference's tests (``tests/golden``) and
against NumPy/SciPy, which those tests use as their own oracle.  For
exp/log/erf the reference's arithmetic lives in oneMKL VM / the SYCL device
library: at the 2-ulp level PARITY IS UNPINNED; the tests bound the CUDA
results against correctly rounded values (mpmath) instead.
"""

from __future__ import annotations

import ctypes as C
import math
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
CORE_PATH = os.path.join(_HERE, "liboracle_core.so")
REF_PATH = os.path.join(_HERE, "_ref", "libref_strided_iters.so")

_core = None
_ref = None


def core():
    """The C restatement (built by ``make -C oracle`` / ``__graft_entry__.build()``)."""
    global _core
    if _core is None:
        if not os.path.exists(CORE_PATH):
            raise RuntimeError(f"{CORE_PATH} is missing: run `make -C oracle`")
        _core = C.CDLL(CORE_PATH)
    return _core


def ref_strided_iters():
    """The reference's simplifier, or None when it was not built."""
    global _ref
    if _ref is None and os.path.exists(REF_PATH):
        _ref = C.CDLL(REF_PATH)
    return _ref


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


# --------------------------------------------------------------- promotion
def binary_result(op, x1, x2):
    """Elementwise binary op with the reference's promotion rules: NumPy's
    result for same-kind safe promotion (dpnp/tensor/_type_utils.py:218-251), true
    division of integers in the default floating type (:89-107), Python scalars
    weak (NEP 50, :389-426).  The reference's tests take NumPy as the expected
    value (dpnp/tests/tensor/elementwise/test_add.py:49-88)."""
    fn = {"add": np.add, "subtract": np.subtract, "multiply": np.multiply, "divide": np.true_divide,
          "maximum": np.maximum, "minimum": np.minimum, "less": np.less, "less_equal": np.less_equal,
          "greater": np.greater, "greater_equal": np.greater_equal, "equal": np.equal,
          "not_equal": np.not_equal, "logical_and": np.logical_and, "logical_or": np.logical_or,
          "power": np.power, "atan2": np.arctan2, "hypot": np.hypot, "copysign": np.copysign,
          "logaddexp": np.logaddexp, "nextafter": np.nextafter, "bitwise_and": np.bitwise_and,
          "bitwise_or": np.bitwise_or, "bitwise_xor": np.bitwise_xor, "logical_xor": np.logical_xor,
          "bitwise_left_shift": shift_left, "bitwise_right_shift": shift_right,
          "floor_divide": floor_divide, "remainder": remainder}[op]
    with np.errstate(all="ignore"):
        return fn(x1, x2)


def shift_left(x1, x2):
    """include/kernels/elementwise_functions/bitwise_left_shift.hpp:88-104: a negative count or
    one of at least the bit width gives 0."""
    x1, x2 = np.asarray(x1), np.asarray(x2)
    bits = x1.dtype.itemsize * 8
    ok = (x2 >= 0) & (x2 < bits)
    return np.where(ok, np.left_shift(x1, np.where(ok, x2, 0).astype(x1.dtype)), 0).astype(x1.dtype)


def shift_right(x1, x2):
    """bitwise_right_shift.hpp:87-105: as above, but a negative value shifted out entirely gives -1."""
    x1, x2 = np.asarray(x1), np.asarray(x2)
    bits = x1.dtype.itemsize * 8
    ok = (x2 >= 0) & (x2 < bits)
    over = np.where((x2 >= bits) & (x1 < 0), -1, 0) if x1.dtype.kind == "i" else 0
    return np.where(ok, np.right_shift(x1, np.where(ok, x2, 0).astype(x1.dtype)), over).astype(x1.dtype)


def floor_divide(x1, x2):
    """floor_divide.hpp:67-90: integers floor towards minus infinity and give 0 for a zero
    divisor; floating types give floor(x1 / x2), keeping a zero quotient as it is."""
    x1, x2 = np.asarray(x1), np.asarray(x2)
    with np.errstate(all="ignore"):
        if x1.dtype.kind in "iu":
            return np.where(x2 == 0, 0, np.floor_divide(x1, np.where(x2 == 0, 1, x2))).astype(x1.dtype)
        ct = np.float32 if x1.dtype == np.float16 else x1.dtype.type
        q = x1.astype(ct) / x2.astype(ct)
        return np.where(q == 0, q, np.floor(q)).astype(x1.dtype)


def remainder(x1, x2):
    """remainder.hpp:66-100: the result takes the sign of the divisor; fmod-based for floats."""
    x1, x2 = np.asarray(x1), np.asarray(x2)
    with np.errstate(all="ignore"):
        if x1.dtype.kind in "iu":
            return np.where(x2 == 0, 0, np.remainder(x1, np.where(x2 == 0, 1, x2))).astype(x1.dtype)
        ct = np.float32 if x1.dtype == np.float16 else x1.dtype.type
        a, b = x1.astype(ct), x2.astype(ct)
        r = np.fmod(a, b)
        adj = (r != 0) & ((b < 0) != (r < 0))
        r = np.where(adj, r + b, r)
        r = np.where(r == 0, np.copysign(ct(0), b), r)
        r = np.where(np.isnan(np.fmod(a, b)), np.fmod(a, b), r)
        return r.astype(x1.dtype)


def unary_result(op, x):
    """Elementwise unary op (include/kernels/elementwise_functions/<op>.hpp).  erf
    follows dpnp/backend/kernels/elementwise_functions/erf.hpp:51-99 (float16 -> float32)."""
    if op == "erf":
        import scipy.special as sp

        if x.dtype == np.float16:
            return sp.erf(x.astype(np.float32))
        return sp.erf(x)
    if op in ("round", "trunc", "floor", "ceil") and x.dtype.kind in "iu":
        return x.copy()                      # identity on integers (round.hpp:70-76, trunc.hpp)
    fn = {"exp": np.exp, "log": np.log, "sqrt": np.sqrt, "negative": np.negative, "abs": np.abs,
          "square": np.square, "sin": np.sin, "cos": np.cos, "tanh": np.tanh, "expm1": np.expm1,
          "log1p": np.log1p, "floor": np.floor, "ceil": np.ceil, "sign": np.sign,
          "reciprocal": np.reciprocal, "positive": np.positive, "logical_not": np.logical_not,
          "isnan": np.isnan, "isinf": np.isinf, "isfinite": np.isfinite,
          "acos": np.arccos, "acosh": np.arccosh, "asin": np.arcsin, "asinh": np.arcsinh,
          "atan": np.arctan, "atanh": np.arctanh, "cbrt": np.cbrt, "cosh": np.cosh, "sinh": np.sinh,
          "tan": np.tan, "exp2": np.exp2, "log2": np.log2, "log10": np.log10,
          "rsqrt": lambda v: (1 / np.sqrt(v)).astype(v.dtype), "trunc": np.trunc, "round": np.rint,
          "signbit": np.signbit, "bitwise_invert": np.invert, "conj": np.conj, "real": np.real,
          "imag": np.imag, "angle": np.angle,
          "proj": proj}[op]
    with np.errstate(all="ignore"):
        return fn(x)


def proj(v):
    """include/kernels/elementwise_functions/proj.hpp: infinite values (either part) map to
    (inf, +-0 with the sign of the imaginary part), everything else is unchanged."""
    v = np.asarray(v)
    out = v.copy()
    m = np.isinf(v.real) | np.isinf(v.imag)
    out.real[m] = np.inf
    out.imag[m] = np.copysign(0.0, v.imag[m])
    return out


def where(cond, x1, x2):
    """dst = cond ? x1 : x2, any non-zero condition is true (include/kernels/where.hpp:108-110)."""
    return np.where(np.asarray(cond) != 0, x1, x2)


# -------------------------------------------------------------- reductions
def default_accumulation_dtype(dt):
    """dpnp/tensor/_type_utils.py:932-952."""
    dt = np.dtype(dt)
    if dt.kind in "bi":
        return np.dtype("i8")
    if dt.kind == "u":
        return np.dtype("u8")
    return dt


def sum_exact(x, axis=None):
    """(sum, sum of magnitudes) in extended precision: the float128/Kahan oracle.
    np.longdouble is the 80-bit x87 type here (64-bit mantissa)."""
    xl = np.asarray(x, dtype=np.longdouble)
    return np.sum(xl, axis=axis), np.sum(np.abs(xl), axis=axis)


def sum_int(x, axis=None, dtype=None):
    """Integer/bool sums are exact modulo 2^bits in the accumulation type
    (source/reductions/sum.cpp:87-241); bool -> bool is logical or (:268-270)."""
    x = np.asarray(x)
    dt = default_accumulation_dtype(x.dtype) if dtype is None else np.dtype(dtype)
    if dt == np.bool_:
        return np.any(x != 0, axis=axis)
    return np.sum(x, axis=axis, dtype=dt)


def max_(x, axis=None, keepdims=False):
    """NaN-propagating maximum (include/utils/sycl_utils.hpp:332-352) == np.max."""
    if np.asarray(x).dtype.kind == "c":
        return complex_extreme(x, axis, True, keepdims)[0]
    return np.max(x, axis=axis, keepdims=keepdims)


def min_(x, axis=None, keepdims=False):
    if np.asarray(x).dtype.kind == "c":
        return complex_extreme(x, axis, False, keepdims)[0]
    return np.min(x, axis=axis, keepdims=keepdims)


def _has_nan(z):
    return z.real != z.real or z.imag != z.imag


def _complex_better(val, best, want_max):
    """greater_complex / less_complex of include/utils/math_utils.hpp:43-69: real parts decide
    unless equal, then imaginary parts; any comparison against a NaN part is false."""
    if val.real == best.real:
        return val.imag > best.imag if want_max else val.imag < best.imag
    if val.imag != val.imag or best.imag != best.imag:
        return False
    return val.real > best.real if want_max else val.real < best.real


def complex_extreme(x, axis=None, want_max=True, keepdims=False):
    """(values, positions) of max/min of a complex array, folding each reduced lane from the
    left with the reference's rules: max_complex / min_complex keep the running value when
    it holds a NaN or wins the comparison, else take the new one
    (include/utils/math_utils.hpp:100-131); the search kernels replace the running value when
    the new one wins or holds a NaN and the running one does not -- a lane's first NaN stays
    (include/kernels/reductions.hpp:1914-1963 with the first-occurrence tie rule of
    :2062-2117).  Pure-Python loops: for small arrays."""
    x = np.asarray(x)
    if axis is None:
        lanes = x.reshape(1, -1)
        out_shape = (1,) * x.ndim if keepdims else ()
    else:
        axes = tuple(sorted(a % x.ndim for a in (axis if isinstance(axis, (tuple, list)) else (axis,))))
        rest = [i for i in range(x.ndim) if i not in axes]
        moved = np.transpose(x, rest + list(axes))
        kept = moved.shape[:len(rest)]
        lanes = np.ascontiguousarray(moved).reshape(int(np.prod(kept, dtype=np.int64)), -1)
        out_shape = tuple(1 if i in axes else x.shape[i] for i in range(x.ndim)) if keepdims else kept
    vals = np.empty(lanes.shape[0], dtype=x.dtype)
    pos = np.empty(lanes.shape[0], dtype=np.int64)
    for r in range(lanes.shape[0]):
        best, at = lanes[r, 0], 0
        for m in range(1, lanes.shape[1]):
            v = lanes[r, m]
            if _has_nan(best):
                break
            if _has_nan(v) or _complex_better(v, best, want_max):
                best, at = v, m
        vals[r], pos[r] = best, at
    return vals.reshape(out_shape), pos.reshape(out_shape)


def argmax(x, axis=None):
    """First occurrence of the maximum, NaN is the maximum
    (include/kernels/reductions.hpp:1933-1963,2062-2117) == np.argmax."""
    if np.asarray(x).dtype.kind == "c":
        return complex_extreme(x, axis, True)[1]
    return np.argmax(x, axis=axis)


def argmin(x, axis=None):
    if np.asarray(x).dtype.kind == "c":
        return complex_extreme(x, axis, False)[1]
    return np.argmin(x, axis=axis)


def mean(x, axis=None):
    """sum in the result type, then one division (dpnp/tensor/_statistical_functions.py:216-269).
    Computed here in extended precision; compare with a tolerance."""
    x = np.asarray(x)
    res_dt = x.dtype if x.dtype.kind in "fc" else np.dtype("f8")
    return np.mean(np.asarray(x, dtype=np.longdouble), axis=axis).astype(res_dt)


# ------------------------------------------------------------ Black-Scholes
def black_scholes_chain(price, strike, t, rate, vol, xp=np, erf=None):
    """The expression chain of examples/example_bs.py:50-75 with array module `xp`."""
    if erf is None:
        import scipy.special as sp

        erf = sp.erf
    mr = -rate
    sig_sig_two = vol * vol * 2
    a = xp.log(price / strike)
    b = t * mr
    z = t * sig_sig_two
    c = 0.25 * z
    y = 1.0 / xp.sqrt(z)
    w1 = (a - b + c) * y
    w2 = (a - b - c) * y
    d1 = 0.5 + 0.5 * erf(w1)
    d2 = 0.5 + 0.5 * erf(w2)
    se = xp.exp(b) * strike
    r = price * d1 - se * d2
    return r, r - price + se


def black_scholes_c(price, strike, t, rate, vol, threads=False):
    """Same chain through the C restatement (libm), optionally on all cores."""
    n = price.size
    call = np.empty(n)
    put = np.empty(n)
    fn = core().orc_black_scholes_f64_mt if threads else core().orc_black_scholes_f64
    fn(C.c_int64(n), _p(price), _p(strike), _p(t), C.c_double(rate), C.c_double(vol), _p(call), _p(put))
    return call, put


# ------------------------------------------------------- iteration spaces
def simplify_ref(shape, strides_list):
    """Collapse with the reference's own code; returns (shape, strides_list, offsets)."""
    lib = ref_strided_iters()
    if lib is None:
        raise RuntimeError("oracle/_ref is not built")
    nd, k = len(shape), len(strides_list)
    sh = (C.c_int64 * max(nd, 1))(*shape)
    st = (C.c_int64 * max(nd * k, 1))(*[s for row in strides_list for s in row])
    off = (C.c_int64 * 4)()
    m = lib.ref_simplify(k, nd, sh, st, off)
    return list(sh[:m]), [list(st[a * nd:a * nd + m]) for a in range(k)], list(off[:k])


def displacement_set(shape, strides_list, offsets=None):
    """Set of displacement tuples visited by an iteration space (brute force)."""
    import itertools

    offsets = offsets or [0] * len(strides_list)
    out = set()
    for idx in itertools.product(*[range(s) for s in shape]):
        out.add(tuple(o + sum(i * s for i, s in zip(idx, st)) for st, o in zip(strides_list, offsets)))
    return out


# --------------------------------------------------------------------- ulp
def ulp_distance(got, exact_longdouble):
    """|got - exact| in units of the last place of `got`'s type at `exact`."""
    got = np.asarray(got)
    ex = np.asarray(exact_longdouble, dtype=np.longdouble)
    spacing = np.spacing(np.abs(ex).astype(got.dtype)).astype(np.longdouble)
    return np.abs(got.astype(np.longdouble) - ex) / spacing


def mp_reference(fn_name, x, digits=40):
    """Correctly rounded reference values of exp/log/erf at the points x, as longdouble."""
    import mpmath

    mpmath.mp.dps = digits
    f = {"exp": mpmath.exp, "log": mpmath.log, "erf": mpmath.erf, "sqrt": mpmath.sqrt}[fn_name]
    out = np.empty(len(x), dtype=np.longdouble)
    for i, v in enumerate(np.asarray(x, dtype=np.float64)):
        out[i] = np.longdouble(mpmath.nstr(f(mpmath.mpf(float(v))), 25))
    return out
