"""Writes tests/golden/known_answers.npz + known_answers.json.

The reference cannot be imported here (it needs dpctl and a SYCL runtime), so
the golden vectors are the known-answer cases of the reference's OWN tests, read
as text: each case rebuilds the input exactly as the test describes it and takes
the expected value from what the test asserts (a literal matrix, a constant, or
a slice of the input) -- never from the operation under test.  ``source`` cites
the test (path relative to the root of IntelPython/dpnp).

Run from the repository root:  python tests/golden/make_golden.py
"""

from __future__ import annotations

import hashlib
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
arrays: dict[str, np.ndarray] = {}
cases: list[dict] = []
_stored_inputs: dict[tuple, str] = {}


def case(name, source, op, x, expected, *, view=None, exact=True, **params):
    """Register one case.  `view` = list of ("flip", axis) / ("slice", spec) /
    ("permute", axes) / ("reshape", shape) steps applied to the stored input before the op."""
    x = np.ascontiguousarray(x)
    digest = (x.dtype.str, x.shape, hashlib.sha1(x.tobytes()).hexdigest())
    entry = {"name": name, "source": source, "op": op, "view": view or [], "exact": exact, "params": params}
    if x.nbytes >= 256 and digest in _stored_inputs:
        entry["x_from"] = _stored_inputs[digest]     # the same input as an earlier case: stored once
    else:
        arrays[f"{name}__x"] = x
        _stored_inputs[digest] = name
    arrays[f"{name}__expected"] = np.asarray(expected)
    cases.append(entry)


T_SUM = "dpnp/tests/tensor/test_tensor_sum.py"
T_RED = "dpnp/tests/tensor/test_usm_ndarray_reductions.py"
T_STAT = "dpnp/tests/tensor/test_tensor_statistical_functions.py"
T_ADD = "dpnp/tests/tensor/elementwise/test_add.py"
T_EXP = "dpnp/tests/tensor/elementwise/test_exp.py"
T_SPECIAL = "dpnp/tests/test_special.py"

# ---- sums -------------------------------------------------------------------
x = np.arange(60, dtype="f4").reshape(3, 4, 5)
case("sum_axis0_3x4x5", f"{T_SUM}:230-247", "sum", x,
     np.array([[60, 63, 66, 69, 72], [75, 78, 81, 84, 87], [90, 93, 96, 99, 102],
               [105, 108, 111, 114, 117]], dtype="f4"), axis=0)
case("sum_flipped_axis2_3x4x5", f"{T_SUM}:249-258", "sum", x,
     np.array([[10, 35, 60, 85], [110, 135, 160, 185], [210, 235, 260, 285]], dtype="f4"),
     view=[["flip", 2]], axis=2)
for n in (1023, 1024, 1025):
    for dt, res_dt in (("i8", "i8"), ("f4", "f4")):
        ones = np.ones((5, n, 5), dtype=dt)
        case(f"sum_ones_5x{n}x5_{dt}_axes01", f"{T_SUM}:184-198", "sum", ones,
             np.full((5,), n * 5, dtype=res_dt), axis=[0, 1])
        case(f"sum_ones_5x{n}x5_{dt}_axes12", f"{T_SUM}:184-198", "sum", ones,
             np.full((5,), n * 5, dtype=res_dt), axis=[1, 2])
    case(f"sum_ones_25x{n}_axis1", f"{T_SUM}:201-212", "sum", np.ones((25, n), dtype="f4"),
         np.full((25,), n, dtype="f4"), axis=1)
    case(f"sum_ones_{n}x25_axis0", f"{T_SUM}:201-212", "sum", np.ones((n, 25), dtype="f4"),
         np.full((25,), n, dtype="f4"), axis=0)
case("sum_gh1391_permuted", f"{T_SUM}:215-227", "sum", np.arange(6, dtype="i4").reshape(1, 2, 3),
     np.array([[0, 3], [1, 4], [2, 5]], dtype="i8"), view=[["permute", [2, 1, 0]]], axis=2)
case("sum_gh1468_int32_to_f4", f"{T_SUM}:328-334", "sum", np.full((2, 3, 4), 123456789, dtype="i4"),
     np.float32(24 * 123456789), exact=False, dtype="f4")
for dt in ("i1", "i2", "i4", "i8", "f2", "f4", "f8"):
    case(f"sum_gh1944_bool_{dt}", f"{T_SUM}:337-348", "sum", np.array([-1, 1], dtype=dt), np.bool_(True),
         dtype="?")

# ---- max / min ----------------------------------------------------------------
x = np.arange(3 * 4 * 5 * 6 * 7, dtype="i4").reshape(3, 4, 5, 6, 7)
case("max_axes_1_2_last", f"{T_RED}:64-75", "max", x, x[:, -1, -1, :, -1], axis=[1, 2, -1])
case("min_axes_1_2_last", f"{T_RED}:77-79", "min", x, x[:, 0, 0, :, 0], axis=[1, 2, -1])
x = np.arange(60, dtype="i8").reshape(3, 4, 5)
case("max_axis0_3x4x5", f"{T_RED}:82-90", "max", x, x[-1, :, :], axis=0)
case("max_flipped_axis2", f"{T_RED}:91-93", "max", x, x[:, :, ::-1][:, :, 0], view=[["flip", 2]], axis=2)
for dt in ("i4", "f4"):
    p = np.ones((24, 1025), dtype=dt)
    p[12, :] = 3
    p[:, 512] = 3
    case(f"max_planted_all_{dt}", f"{T_RED}:119-133", "max", p, np.asarray(3, dtype=dt), axis=None)
    case(f"max_planted_axis0_{dt}", f"{T_RED}:119-133", "max", p, np.full(1025, 3, dtype=dt), axis=0)
    case(f"max_planted_axis1_{dt}", f"{T_RED}:119-133", "max", p, np.full(24, 3, dtype=dt), axis=1)
    p = np.ones((24, 1025), dtype=dt)
    p[12, :] = 0
    p[:, 512] = 0
    case(f"min_planted_all_{dt}", f"{T_RED}:135-147", "min", p, np.asarray(0, dtype=dt), axis=None)
    case(f"min_planted_axis0_{dt}", f"{T_RED}:135-147", "min", p, np.full(1025, 0, dtype=dt), axis=0)
    case(f"min_planted_axis1_{dt}", f"{T_RED}:135-147", "min", p, np.full(24, 0, dtype=dt), axis=1)
x = np.arange(4, dtype="f4")
x[0] = np.nan
case("max_nan_finite", f"{T_RED}:150-157", "max", x, np.float32(np.nan), axis=None)
case("min_nan_finite", f"{T_RED}:150-157", "min", x, np.float32(np.nan), axis=None)
x = x.copy()
x[1:] = np.inf
case("max_nan_inf", f"{T_RED}:159-161", "max", x, np.float32(np.nan), axis=None)
x = x.copy()
x[1:] = -np.inf
case("min_nan_neginf", f"{T_RED}:162-163", "min", x, np.float32(np.nan), axis=None)

# ---- argmax / argmin ------------------------------------------------------------
# the reference test draws `idx` with randrange; fixed positions are used here
shape = (24, 1024)
size = shape[0] * shape[1]
for dt in ("i4", "f4"):
    for tag, idx in (("a", 7777), ("b", 0), ("c", size - 1)):
        x = np.ones(size, dtype=dt)
        x[idx] = 2
        case(f"argmax_planted_flat_{dt}_{tag}", f"{T_RED}:186-201", "argmax", x, np.int64(idx), axis=None)
        case(f"argmax_planted_flipped_{dt}_{tag}", f"{T_RED}:203-206", "argmax", x,
             np.int64(size - 1 - idx), view=[["flip", 0]], axis=None)
        y = np.ones(2 * size, dtype=dt)
        y[::2] = x
        case(f"argmax_planted_strided_{dt}_{tag}", f"{T_RED}:208-212", "argmax", y, np.int64(idx),
             view=[["slice", [[None, None, 2]]]], axis=None)
    idx = 7777
    r, c = np.unravel_index(idx, shape)
    x = np.ones(size, dtype=dt)
    x[idx] = 2
    x = x.reshape(shape)
    x[r, :] = 3
    case(f"argmax_planted_axis0_{dt}", f"{T_RED}:214-218", "argmax", x, np.full(1024, r, dtype="i8"), axis=0)
    x = x.copy()
    x[:, c] = 4
    case(f"argmax_planted_axis1_{dt}", f"{T_RED}:219-221", "argmax", x, np.full(24, c, dtype="i8"), axis=1)
    xs = x.copy()
    j = 300  # position inside the reversed, every-second-column view
    xs[:, ::-2][:, j] = 5
    case(f"argmax_planted_negstride_{dt}", f"{T_RED}:223-227", "argmax", xs, np.full(24, j, dtype="i8"),
         view=[["slice", [[None, None, None], [None, None, -2]]]], axis=1)
    x = np.ones(size, dtype=dt)
    x[idx] = 0
    case(f"argmin_planted_flat_{dt}", f"{T_RED}:229-235", "argmin", x, np.int64(idx), axis=None)
    x = x.reshape(shape).copy()
    x[r, :] = -1
    case(f"argmin_planted_axis0_{dt}", f"{T_RED}:237-241", "argmin", x, np.full(1024, r, dtype="i8"), axis=0)
    x = x.copy()
    x[:, c] = -2
    case(f"argmin_planted_axis1_{dt}", f"{T_RED}:242-244", "argmin", x, np.full(24, c, dtype="i8"), axis=1)
for idx in range(4):
    x = np.arange(4, dtype="f4")
    x[idx] = np.nan
    case(f"argmax_nan_at_{idx}", f"{T_RED}:254-262", "argmax", x, np.int64(idx), axis=None)
    case(f"argmin_nan_at_{idx}", f"{T_RED}:254-262", "argmin", x, np.int64(idx), axis=None)
case("argmax_all_int32_min", f"{T_RED}:276-281", "argmax", np.full(3, np.iinfo("i4").min, dtype="i4"),
     np.int64(0), axis=None)
case("argmin_all_int32_max", f"{T_RED}:282-283", "argmin", np.full(3, np.iinfo("i4").max, dtype="i4"),
     np.int64(0), axis=None)
x = np.array([[1, 2, 3], [6, 5, 4]], dtype="i4")
for order in ("C", "F"):
    case(f"argmax_2x3_flat_{order}", f"{T_RED}:286-291", "argmax", x, np.int64(3), axis=None, order=order)
    case(f"argmax_2x3_axis0_{order}", f"{T_RED}:293-295", "argmax", x, np.array([1, 1, 1], dtype="i8"),
         axis=0, order=order)
    case(f"argmax_2x3_axis1_{order}", f"{T_RED}:297-299", "argmax", x, np.array([2, 0], dtype="i8"),
         axis=1, order=order)
case("argmax_0d", f"{T_RED}:176-183", "argmax", np.ones((), dtype="f8"), np.int64(0), axis=None)

# ---- mean -----------------------------------------------------------------------
x = np.arange(9, dtype="f4").reshape(3, 3)
case("mean_3x3_all", f"{T_STAT}:159-173", "mean", x, np.float32(4), axis=None)
case("mean_3x3_axis0", f"{T_STAT}:159-173", "mean", x, np.array([3, 4, 5], dtype="f4"), axis=0)
case("mean_3x3_axis1", f"{T_STAT}:159-173", "mean", x, np.array([1, 4, 7], dtype="f4"), axis=1)
case("mean_empty_is_nan", f"{T_STAT}:107-122", "mean", np.empty((10, 0, 5), dtype="f4"),
     np.full((10, 5), np.nan, dtype="f4"), axis=1)

# ---- add with broadcasting ----------------------------------------------------------
m = np.ones((100, 5), dtype="i4")
v = np.arange(5, dtype="i4")
arrays["add_bcast_100x5__y"] = v
case("add_bcast_100x5", f"{T_ADD}:139-157", "add", m,
     np.broadcast_to(np.arange(1, 6, dtype="i4")[np.newaxis, :], (100, 5)).copy())
arrays["add_bcast_6x1_6__y"] = np.arange(6, dtype="i4")
case("add_bcast_6x1_6", f"{T_ADD}:160-168", "add", np.ones((6, 1), dtype="i4"),
     np.broadcast_to(np.arange(1, 7, dtype="i4")[np.newaxis, :], (6, 6)).copy())
arrays["add_bcast_6x1_1x6__y"] = np.ones((1, 6), dtype="i4")
case("add_bcast_6x1_1x6", f"{T_ADD}:182-190", "add", np.ones((6, 1), dtype="i4"), np.full((6, 6), 2, dtype="i4"))

# ---- exp / erf special values --------------------------------------------------------
log2_ = 0.69314718055994530943
for dt in ("f4", "f8"):
    xs = np.array([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10], dtype=dt) * np.asarray(log2_, dtype=dt)
    case(f"exp_k_ln2_{dt}", f"{T_EXP}:110-120", "exp", xs, (2.0 ** np.arange(11)).astype(dt), exact=False)
    case(f"exp_special_{dt}", f"{T_EXP}:123-137", "exp", np.array([np.nan, np.inf, -np.inf, 0.0, -0.0], dtype=dt),
         np.array([np.nan, np.inf, 0.0, 1.0, 1.0], dtype=dt))
case("erf_nan_inf", f"{T_SPECIAL}:38-46", "erf", np.array([np.nan, -np.inf, np.inf]), np.array([np.nan, -1.0, 1.0]))
case("erf_zeros_signbit", f"{T_SPECIAL}:48-57", "erf", np.array([0.0, -0.0]), np.array([0.0, -0.0]))

# ---- where -----------------------------------------------------------------------------
T_WHERE = "dpnp/tests/tensor/test_usm_ndarray_search_functions.py"


def where_case(name, source, cond, x1, x2, expected, *, views=None, exact=True):
    """`views` maps "cond"/"x"/"y" to view steps applied to the stored operand before the call."""
    arrays[f"{name}__cond"] = np.ascontiguousarray(cond)
    arrays[f"{name}__y"] = np.ascontiguousarray(x2)
    case(name, source, "where", x1, expected, exact=exact, views=views or {})


cond = np.array([[True, False, False], [False, True, False], [False, False, True],
                 [False, False, False], [True, True, True]])
eye_like = np.array([[1, 0, 0], [0, 1, 0], [0, 0, 1], [0, 0, 0], [1, 1, 1]])
where_case("where_basic_0d_operands", f"{T_WHERE}:69-86", cond, np.asarray(1), np.asarray(0), eye_like)
where_case("where_basic_full_operands", f"{T_WHERE}:88-89", cond, np.ones(cond.shape), np.zeros(cond.shape),
           eye_like.astype("f8"))
where_case("where_basic_column_operands", f"{T_WHERE}:91-96", cond, np.ones((5, 1), dtype="i4"),
           np.zeros((5, 1), dtype="i4"), eye_like.astype("i4"))
c4 = np.array([True, False, True, False])
a4 = np.array([np.nan, 2.0, np.inf, 3.0], dtype="f4")
b4 = np.array([2.0, np.nan, 3.0, np.inf], dtype="f4")
# expected values written out element by element: cond ? x1 : x2
where_case("where_nan_inf", f"{T_WHERE}:189-203", c4, a4, b4, np.array([np.nan, np.nan, np.inf, np.inf], dtype="f4"))
# a floating condition: NaN and inf are non-zero, hence true; bool and float32 promote to float32
where_case("where_float_condition", f"{T_WHERE}:205-207", a4, c4, b4, np.array([1.0, 0.0, 1.0, 0.0], dtype="f4"))
s0, s1 = 4, 9
cond_full = np.array([True, False, False, False, True, True, False, True, False] * s0).reshape(s0, s1)
x1_full = np.arange(s0 * 3 * 2, dtype="i4").reshape(s0, 6)
x2_full = np.arange(s0 * 3 * 3, dtype="i4").reshape(s0, 9)
cv, xv, yv = cond_full[:, ::3], x1_full[:, ::2], x2_full[:, ::3]
sl3, sl2 = [[None, None, None], [None, None, 3]], [[None, None, None], [None, None, 2]]


def pick(c_, a_, b_):
    out = np.empty(c_.shape, dtype=a_.dtype)
    for idx in np.ndindex(*c_.shape):
        out[idx] = a_[idx] if c_[idx] else b_[idx]
    return out


where_case("where_strided", f"{T_WHERE}:294-313", cond_full, x1_full, x2_full, pick(cv, xv, yv),
           views={"cond": [["slice", sl3]], "x": [["slice", sl2]], "y": [["slice", sl3]]})
where_case("where_strided_flipped_x1", f"{T_WHERE}:315-320", cond_full, x1_full, x2_full,
           pick(cv, xv[::-1, ::-1], yv),
           views={"cond": [["slice", sl3]], "x": [["slice", sl2], ["flip", None]], "y": [["slice", sl3]]})
where_case("where_strided_flipped_cond", f"{T_WHERE}:322-326", cond_full, x1_full, x2_full,
           pick(cv[::-1, ::-1], xv, yv),
           views={"cond": [["slice", sl3], ["flip", None]], "x": [["slice", sl2]], "y": [["slice", sl3]]})
where_case("where_unaligned", f"{T_WHERE}:451-461", np.ones(513, dtype="i4"), np.full(512, 2, dtype="i4"),
           np.zeros(512, dtype="i4"), np.full(512, 2, dtype="i4"), views={"cond": [["slice", [[1, None, None]]]]})

# ---- the ported CuPy reduction suite: max/min/argmax/argmin against NumPy ------------------
# Its inputs come from testing.shaped_random (RandomState(0).rand(*shape) * 10 cast to the type;
# booleans from randint(2); complex from two draws) in C and F order, and its expected value is
# NumPy's result on the same input (testing.numpy_cupy_allclose), which is what is stored here.
T_CUPY = "dpnp/tests/third_party/cupy/core_tests/test_ndarray_reduction.py"


def shaped_random(shape, dtype, scale=10, seed=0):
    rng = np.random.RandomState(seed)
    dtype = np.dtype(dtype)
    if dtype == "?":
        a = rng.randint(2, size=shape)
    elif dtype.kind == "c":
        a = rng.rand(*shape) + 1j * rng.rand(*shape)
        a *= scale
    else:
        a = rng.rand(*shape) * scale
    return np.asarray(a, dtype=dtype)


ALL_DTYPES = ("?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8", "f2", "f4", "f8", "c8", "c16")
CUPY_SHAPES = [  # (tag, lines for max / min / argmax / argmin, shape, axis, keepdims)
    ("all", (45, 119, 193, 249), (2, 3), None, False),
    ("all_keepdims", (51, 125, None, None), (2, 3), None, True),
    ("axis_large", (57, 131, 199, 255), (3, 1000), 0, False),
    ("axis0", (63, 137, 205, 261), (2, 3, 4), 0, False),
    ("axis1", (69, 143, 211, 267), (2, 3, 4), 1, False),
    ("axis2", (75, 149, 217, 273), (2, 3, 4), 2, False),
    ("multiple_axes", (81, 155, None, None), (2, 3, 4), [1, 2], False),
    ("multiple_axes_keepdims", (87, 161, None, None), (2, 3, 4), [1, 2], True),
]
for fn_i, fn in enumerate(("max", "min", "argmax", "argmin")):
    for tag, lines, shape, axis, keepdims in CUPY_SHAPES:
        if lines[fn_i] is None:
            continue
        for dt in ALL_DTYPES:
            a = shaped_random(shape, dt)
            ax = tuple(axis) if isinstance(axis, list) else axis
            kw = {"keepdims": True} if keepdims else {}
            want = getattr(np, fn)(a, axis=ax, **kw)
            for order in ("C", "F"):
                case(f"cupy_{fn}_{tag}_{np.dtype(dt).name}_{order}", f"{T_CUPY}:{lines[fn_i]}-{lines[fn_i] + 4}",
                     fn, a, want, axis=axis, order=order, **kw)
    first = {"max": 93, "min": 167, "argmax": 223, "argmin": 279}[fn]
    for order in ("C", "F"):
        for dt in ("f2", "f4", "f8"):
            a = np.array([float("nan"), 1, -1], dt)
            case(f"cupy_{fn}_nan_{np.dtype(dt).name}_{order}", f"{T_CUPY}:{first}-{first + 4}", fn, a,
                 getattr(np, fn)(a), axis=None, order=order)
            if fn in ("max", "min"):
                inf = -float("inf") if fn == "max" else float("inf")
                a = np.array([inf, inf], dt)
                case(f"cupy_{fn}_inf_{np.dtype(dt).name}_{order}", f"{T_CUPY}:{first + 18}-{first + 23}", fn, a,
                     getattr(np, fn)(a), axis=None, order=order)
        for dt in ("c8", "c16"):
            a = np.array([float("nan"), 1, -1], dt)
            case(f"cupy_{fn}_nan_real_{np.dtype(dt).name}_{order}", f"{T_CUPY}:{first + 6}-{first + 10}", fn, a,
                 getattr(np, fn)(a), axis=None, order=order)
            a = np.array([float("nan") * 1.0j, 1.0j, -1.0j], dt)
            case(f"cupy_{fn}_nan_imag_{np.dtype(dt).name}_{order}", f"{T_CUPY}:{first + 12}-{first + 16}", fn, a,
                 getattr(np, fn)(a), axis=None, order=order)

np.savez_compressed(os.path.join(HERE, "known_answers.npz"), **arrays)
with open(os.path.join(HERE, "known_answers.json"), "w") as fh:
    json.dump(cases, fh, indent=1)
print(f"{len(cases)} cases, {sum(a.nbytes for a in arrays.values()) / 1e6:.1f} MB raw")
