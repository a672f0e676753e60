"""The rest of the elementwise family (inverse trigonometric, hyperbolic, base-2/10, rounding,
bit operations, floor division and remainder, complex parts) against the CPU oracle.

Integer and bit results, rounding functions, copysign, nextafter, signbit and the complex-part
functions are bit-exact.  Floating-point functions are compared with NumPy within 4 ulp (each
side is within 2 ulp of the exact value)."""

import zlib

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu

INTS = ["i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8"]
FLOATS = ["f2", "f4", "f8"]


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


def ulps(got, ref):
    got, ref = np.asarray(got), np.asarray(ref)
    fin = np.isfinite(ref) & np.isfinite(got)
    assert np.array_equal(np.isnan(got), np.isnan(ref))
    assert np.array_equal(got[~fin & ~np.isnan(ref)], ref[~fin & ~np.isnan(ref)])
    if not fin.any():
        return 0.0
    sp = np.spacing(np.abs(ref[fin]).astype(ref.dtype)).astype("f8")
    return float(np.max(np.abs(got[fin].astype("f8") - ref[fin].astype("f8")) / sp))


def assert_same_bits(got, ref, what=""):
    """Bit equality, except that any NaN matches any NaN (the payload a NaN result carries is
    not part of the contract)."""
    got, ref = np.ascontiguousarray(got), np.ascontiguousarray(ref)
    assert got.dtype == ref.dtype and got.shape == ref.shape, what
    if got.dtype.kind == "c":
        rt = got.real.dtype
        got, ref = got.view(rt), ref.view(rt)
    if got.dtype.kind == "f":
        nan = np.isnan(ref)
        assert np.array_equal(np.isnan(got), nan), what
        got, ref = got[~nan], ref[~nan]
    np.testing.assert_array_equal(got.view(np.uint8), ref.view(np.uint8), err_msg=what)


DOMAINS = {"acos": (-1, 1), "asin": (-1, 1), "acosh": (1, 50), "atanh": (-0.999, 0.999), "log2": (1e-3, 1e3),
           "log10": (1e-3, 1e3), "rsqrt": (1e-3, 1e3), "cosh": (-8, 8), "sinh": (-8, 8), "exp2": (-10, 10),
           "tan": (-1.5, 1.5)}


@pytest.mark.parametrize("dt", FLOATS)
@pytest.mark.parametrize("op", ["acos", "acosh", "asin", "asinh", "atan", "atanh", "cbrt", "cosh", "sinh", "tan",
                                "exp2", "log2", "log10", "rsqrt"])
def test_float_functions(op, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(zlib.crc32(f"{op}{dt}".encode()))
    lo, hi = DOMAINS.get(op, (-20, 20))
    x = rng.uniform(lo, hi, 5000).astype(dt)
    x[:4] = [np.nan, np.inf, -np.inf, 0.0]
    got = getattr(dp.tensor._elementwise_funcs, op)(dev(x).get_array())
    # float16 is evaluated in float32 and rounded once (NumPy's own float16 loops may use
    # lower-accuracy vector routines, so they are not the reference here)
    ref = orc.unary_result(op, x) if dt != "f2" else orc.unary_result(op, x.astype("f4")).astype("f2")
    assert got.dtype == ref.dtype
    limit = 4 if dt != "f2" else 1.01        # float16 is computed in float32 and rounded once
    assert ulps(dp.asnumpy(got), ref) <= limit
    # integers are promoted to the default floating type first
    xi = rng.integers(1, 5, 100).astype("i4")
    gi = getattr(dp, op if hasattr(dp, op) else "arc" + op[1:])(dev(xi))
    with np.errstate(all="ignore"):
        assert gi.dtype == np.dtype("f8") and ulps(gi.asnumpy(), orc.unary_result(op, xi.astype("f8"))) <= 4


@pytest.mark.parametrize("dt", FLOATS + INTS + ["c8", "c16"])
def test_rounding_sign_and_complex_parts_are_exact(dt):
    import dpnp_b200 as dp
    from dpnp_b200.tensor import _elementwise_funcs as ef

    rng = np.random.default_rng(zlib.crc32(dt.encode()))
    k = np.dtype(dt).kind
    if k == "c":
        x = (rng.uniform(-9, 9, 3000) + 1j * rng.uniform(-9, 9, 3000)).astype(dt)
        x[:3] = [complex(np.inf, -1), complex(2, -np.inf), complex(np.nan, 0.0)]
    elif k == "f":
        x = (rng.integers(-40, 40, 3000) / 4).astype(dt)        # plenty of exact halves
        x[:5] = [np.nan, np.inf, -np.inf, -0.0, 0.0]
    else:
        x = rng.integers(0 if k == "u" else -100, 100, 3000).astype(dt)
    d = dev(x).get_array()
    ops = ["round", "conj", "real", "imag"] + ([] if k == "c" else ["trunc"]) + (["signbit"] if k == "f" else []) \
        + (["bitwise_invert"] if k in "iu" else []) + (["angle", "proj"] if k == "c" else [])
    for op in ops:
        got = dp.asnumpy(getattr(ef, op)(d))
        ref = orc.unary_result(op, x)
        assert got.dtype == ref.dtype, (op, got.dtype, ref.dtype)
        if op == "angle":
            assert ulps(got, ref) <= 4
        else:
            assert_same_bits(got, ref, op)
    if k == "c":
        assert ef.trunc.result_type_resolver_fn_(np.dtype(dt)) is None


def test_round_with_decimals():
    """dpnp.round scales, rounds half to even and scales back (dpnp_elementwise_common.py:1317-1341)."""
    import dpnp_b200 as dp

    x = np.array([1.2345, -2.5, 0.125, 37.5, 1234.5678])
    np.testing.assert_allclose(dp.round(dev(x), 2).asnumpy(), np.round(x, 2), rtol=1e-15)
    np.testing.assert_allclose(dp.around(dev(x), -1).asnumpy(), np.round(x, -1), rtol=1e-15)
    np.testing.assert_array_equal(dp.round(dev(x)).asnumpy(), np.round(x))
    xi = np.array([14, 15, 25, -35, 123], dtype="i4")
    np.testing.assert_array_equal(dp.round(dev(xi), 1).asnumpy(), xi)
    out = dp.empty(5)
    assert dp.round(dev(x), 1, out=out) is out
    np.testing.assert_allclose(out.asnumpy(), np.round(x, 1), rtol=1e-15)


def test_bool_inputs_of_round_conj_and_invert():
    import dpnp_b200 as dp
    from dpnp_b200.tensor import _elementwise_funcs as ef

    b = np.array([True, False, True])
    d = dev(b).get_array()
    assert dp.asnumpy(ef.conj(d)).dtype == np.dtype("i1")
    np.testing.assert_array_equal(dp.asnumpy(ef.bitwise_invert(d)), ~b)
    r = ef.round(d)                                   # bool rounds in a floating type
    assert r.dtype.kind == "f"
    np.testing.assert_array_equal(dp.asnumpy(r), b.astype(r.dtype))
    np.testing.assert_array_equal((~dev(b)).asnumpy(), ~b)


@pytest.mark.parametrize("dt", FLOATS)
def test_float_binary_functions(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(zlib.crc32(dt.encode()) + 1)
    x, y = rng.uniform(-30, 30, 4000).astype(dt), rng.uniform(-30, 30, 4000).astype(dt)
    x[:6] = [np.nan, np.inf, -np.inf, 0.0, -0.0, 5.0]
    y[:6] = [1.0, np.inf, np.inf, -0.0, 0.0, np.nan]
    dx, dy = dev(x), dev(y)
    for op in ("atan2", "hypot", "logaddexp"):
        got = getattr(dp, op)(dx, dy).asnumpy()
        ref = orc.binary_result(op, x, y) if dt != "f2" else \
            orc.binary_result(op, x.astype("f4"), y.astype("f4")).astype("f2")
        assert got.dtype == ref.dtype
        assert ulps(got, ref) <= (4 if dt != "f2" else 1.01), op
    for op in ("copysign", "nextafter"):
        got = getattr(dp, op)(dx, dy).asnumpy()
        ref = orc.binary_result(op, x, y)
        if op == "nextafter":
            ref = np.where(x == y, y, ref)             # equal operands give the second one (C rule)
        assert_same_bits(got, ref, op)
    for op, sym in (("floor_divide", "//"), ("remainder", "%")):
        got = getattr(dp, op)(dx, dy).asnumpy()
        ref = orc.binary_result(op, x, y)
        nan = np.isnan(ref)
        assert np.array_equal(np.isnan(got), nan), op
        np.testing.assert_array_equal(got[~nan].view(np.uint8), ref[~nan].view(np.uint8), err_msg=op)
    np.testing.assert_array_equal((dx[6:] // 3).asnumpy(), orc.floor_divide(x[6:], np.full_like(x[6:], 3)))
    np.testing.assert_array_equal((dx[6:] % -7).asnumpy(), orc.remainder(x[6:], np.full_like(x[6:], -7)))


@pytest.mark.parametrize("dt", INTS)
def test_integer_binary_functions_are_exact(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(zlib.crc32(dt.encode()) + 2)
    info = np.iinfo(dt)
    x = rng.integers(info.min, info.max, 4000, dtype=dt, endpoint=True)
    y = rng.integers(info.min, info.max, 4000, dtype=dt, endpoint=True)
    y[:4] = [0, 1, info.max, info.min]
    x[:4] = [info.min, info.min, info.max, info.min]
    if info.min < 0:
        y[4], x[4] = -1, info.min                      # the one quotient that does not fit
    dx, dy = dev(x), dev(y)
    for op in ("bitwise_and", "bitwise_or", "bitwise_xor", "logical_xor"):
        np.testing.assert_array_equal(getattr(dp, op)(dx, dy).asnumpy(), orc.binary_result(op, x, y), err_msg=op)
    sel = np.ones(4000, bool)
    if info.min < 0:
        sel[4] = False                                 # NumPy's own answer for min // -1 is platform-defined
    for op in ("floor_divide", "remainder"):
        got = getattr(dp, op)(dx, dy).asnumpy()
        np.testing.assert_array_equal(got[sel], orc.binary_result(op, x, y)[sel], err_msg=op)
    if info.min < 0:
        assert dp.floor_divide(dx, dy).asnumpy()[4] == info.min and dp.remainder(dx, dy).asnumpy()[4] == 0
    bits = np.dtype(dt).itemsize * 8
    s = rng.integers(-3 if info.min < 0 else 0, bits + 3, 4000).astype(dt)
    ds = dev(s)
    np.testing.assert_array_equal(dp.left_shift(dx, ds).asnumpy(), orc.shift_left(x, s))
    np.testing.assert_array_equal(dp.right_shift(dx, ds).asnumpy(), orc.shift_right(x, s))
    # operators, Python scalars, in-place forms
    np.testing.assert_array_equal((dx & 7).asnumpy(), x & np.dtype(dt).type(7))
    np.testing.assert_array_equal((dx ^ dy).asnumpy(), x ^ y)
    np.testing.assert_array_equal((dx >> 2).asnumpy(), x >> np.dtype(dt).type(2))
    np.testing.assert_array_equal((~dx).asnumpy(), ~x)
    z = dev(x.copy())
    z |= dy
    np.testing.assert_array_equal(z.asnumpy(), x | y)
    z = dev(x.copy())
    z //= 3
    np.testing.assert_array_equal(z.asnumpy(), x // np.dtype(dt).type(3))


def test_type_rules_and_strided_operands():
    import dpnp_b200 as dp

    with pytest.raises((TypeError, ValueError)):
        dp.bitwise_and(dev(np.ones(3)), dev(np.ones(3)))
    # bool operands of a shift are promoted to int8, as every operand without an exact match is
    assert dp.left_shift(dev(np.ones(3, "?")), dev(np.ones(3, "?"))).dtype == np.dtype("i1")
    a = np.arange(-30, 30, dtype="i4").reshape(6, 10)
    b = np.arange(1, 11, dtype="i2")
    np.testing.assert_array_equal((dev(a).T % dev(b)[:6]).asnumpy(), a.T % b[:6].astype("i4"))
    np.testing.assert_array_equal(dp.logical_xor(dev(a)[::2], dev(b)).asnumpy(), np.logical_xor(a[::2], b))
    f = np.linspace(-4, 4, 60).reshape(6, 10)
    got = dp.arctan2(dev(f)[:, ::-1], dev(f).T[:10, :6].T).asnumpy()
    assert ulps(got, np.arctan2(f[:, ::-1], f)) <= 4


# ---- known-answer cases of the reference's own tests (dpnp/tests/tensor/elementwise/); the
# expected values are the literals / NumPy results those tests assert.
def test_reference_floor_divide_cases():
    """test_floor_divide.py:80-147 (gh-1247, zero divisors, special values)."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    x = dp.ones(1, dtype="i4").get_array()
    np.testing.assert_array_equal(dp.asnumpy(dpt.floor_divide(x, -2)), np.full(1, -1, "i4"))
    x = dp.full(1, -1, dtype="i4").get_array()
    np.testing.assert_array_equal(dp.asnumpy(dpt.floor_divide(x, 2)), np.full(1, -1, "i4"))
    for dt in INTS:
        xa = dev(np.arange(10, dtype=dt)).get_array()
        r = dpt.floor_divide(xa, dev(np.zeros(10, dtype=dt)).get_array())
        np.testing.assert_array_equal(dp.asnumpy(r), np.zeros(10, dtype=dt))

    def fd(a, b):
        return dp.asnumpy(dpt.floor_divide(dev(np.array([a], "f4")).get_array(), dev(np.array([b], "f4")).get_array()))

    assert np.isnan(fd(np.inf, np.inf)[0])
    r = fd(0.0, -1.0)
    assert r[0] == 0 and np.signbit(r[0])                     # -0.0
    assert fd(-1.0, 0.0)[0] == -np.inf
    r = fd(-1.0, np.inf)
    assert r[0] == 0 and np.signbit(r[0])                     # the literal the test asserts: -0.0
    assert fd(np.inf, -1.0)[0] == -np.inf
    assert np.isnan(fd(1.0, np.nan)[0])


def test_reference_remainder_cases():
    """test_remainder.py:80-153 (negative integers, zero divisors, negative floats, special values)."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    for dt in ("i1", "i2", "i4", "i8"):
        x_np = np.arange(-5, -1, 1, dtype=dt)
        x = dev(x_np).get_array()
        assert (dp.asnumpy(dpt.remainder(x, 3)) == np.remainder(x_np, 3)).all()
        assert (dp.asnumpy(dpt.remainder(3, x)) == np.remainder(3, x_np)).all()
    for dt in ("i4", "u4"):
        r = dpt.remainder(dp.ones(1, dtype=dt).get_array(), dp.zeros(1, dtype=dt).get_array())
        assert (dp.asnumpy(r) == np.zeros(1, dtype=dt)).all()
    for dt in ("f2", "f4", "f8"):
        x_np = np.linspace(-5, 5, 20, dtype=dt)
        x = dev(x_np).get_array()
        tol = 8 * np.finfo(dt).resolution
        np.testing.assert_allclose(dp.asnumpy(dpt.remainder(x, 3)), np.remainder(x_np, dt and np.dtype(dt).type(3)),
                                   rtol=tol, atol=tol)
        with np.errstate(all="ignore"):
            np.testing.assert_allclose(dp.asnumpy(dpt.remainder(3, x)), np.remainder(np.dtype(dt).type(3), x_np),
                                       rtol=tol, atol=tol)
    lhs = [np.nan, np.inf, 0.0, -0.0, -0.0, 1.0, np.inf, -np.inf]
    rhs = [np.nan, np.inf, -0.0, 1.0, 1.0, 0.0, 1.0, -1.0]
    x_np, y_np = np.asarray(lhs, "f4"), np.asarray(rhs, "f4")
    with np.errstate(all="ignore"):
        np.testing.assert_allclose(dp.asnumpy(dpt.remainder(dev(x_np).get_array(), dev(y_np).get_array())),
                                   np.remainder(x_np, y_np))


def test_reference_shift_round_nextafter_cases():
    """test_bitwise_left_shift.py:107-117 and test_bitwise_right_shift.py (a count of 64 gives 0),
    test_round.py:109-123 (halves to even, signs of zero), test_nextafter.py:80-140."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    for dt in INTS:
        x = dp.ones(255, dtype=dt).get_array()
        y = dev(np.asarray(64, dtype=dt)).get_array()
        assert not dp.asnumpy(dpt.bitwise_left_shift(x, y)).any()
        assert not dp.asnumpy(dpt.bitwise_right_shift(x, y)).any()
    for dt in FLOATS:
        x = np.array([np.nan, np.inf, -np.inf, 1.5, 2.5, -1.5, -2.5, 0.0, -0.0], dtype=dt)
        y = dp.asnumpy(dpt.round(dev(x).get_array()))
        ref = np.round(x)
        np.testing.assert_array_equal(y[1:], ref[1:])
        assert np.isnan(y[0])
        np.testing.assert_array_equal(np.signbit(y[1:]), np.signbit(ref[1:]))
        x1 = dev(np.array([2.0, np.nan, np.nan], dtype=dt)).get_array()
        x2 = dev(np.array([np.nan, 2.0, np.nan], dtype=dt)).get_array()
        assert np.isnan(dp.asnumpy(dpt.nextafter(x1, x2))).all()
        z1 = np.array([-0.0, 0.0, -0.0, 0.0], dtype=dt)
        z2 = np.array([0.0, -0.0, -0.0, 0.0], dtype=dt)
        yz = dp.asnumpy(dpt.nextafter(dev(z1).get_array(), dev(z2).get_array()))
        assert (yz == 0).all()
        np.testing.assert_array_equal(np.signbit(yz), np.signbit(z2))          # equal operands give x2
        ones, twos = dp.ones(10, dtype=dt).get_array(), dp.full(10, 2, dtype=dt).get_array()
        r = dp.asnumpy(dpt.nextafter(ones, twos))
        assert (r > 0).all() and (r - np.ones(10, dt) == np.finfo(dt).eps).all()
        zeros = dp.zeros(10, dtype=dt).get_array()
        assert (dp.asnumpy(dpt.nextafter(zeros, ones)) > 0).all()
        assert ((dp.asnumpy(dpt.nextafter(ones, zeros)) - np.ones(10, dt)) < 0).all()
