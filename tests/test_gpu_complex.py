"""Complex arguments of the elementwise family and integer powers on the device.

Oracle: NumPy on the same inputs, with the tolerances of the reference's own tests
(8 x finfo.resolution on random arguments and special values, tests/tensor/elementwise/
test_exp.py:81-106,215-235; 50 x resolution for the trigonometric / hyperbolic families,
test_trigonometric.py:101-133); the reference's literal expectations for expm1
(test_expm1.py:97-140); bit equality for comparisons, maximum/minimum and integer powers."""

import itertools
import warnings

import numpy as np
import pytest

from tests.test_complex_host import GRID, RES, expected, modulus_close, parts_close

pytestmark = pytest.mark.gpu

NAMES = {"arcsin": "asin", "arccos": "acos", "arctan": "atan", "arcsinh": "asinh", "arccosh": "acosh",
         "arctanh": "atanh"}
UNARY = ["exp", "log", "sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh", "arcsin", "arccos", "arctan",
         "arcsinh", "arccosh", "arctanh", "expm1", "log1p", "log2", "log10", "exp2", "reciprocal", "sign"]


def device(name, z):
    import dpnp_b200 as dp

    return getattr(dp, NAMES.get(name, name))(dp.asarray(z)).asnumpy()


@pytest.mark.parametrize("dt", ["c8", "c16"])
@pytest.mark.parametrize("name", UNARY)
def test_unary_random_special_and_views(name, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(UNARY.index(name))
    ranges = [(-9, 9), (-88, 88)] if name in ("exp", "expm1") else [(-9, 9), (-0.5, 0.5)]
    tol = (50 if name in ("sin", "cos", "tan", "sinh", "cosh", "tanh", "arcsin", "arccos", "arctan", "arcsinh",
                          "arccosh", "arctanh") else 8) * RES[dt]
    for lo, hi in ranges:
        z = (rng.uniform(lo, hi, 5003) + 1j * rng.uniform(lo, hi, 5003)).astype(dt)
        got, exp = device(name, z), expected(name, z)
        assert got.dtype == exp.dtype
        bad = ~parts_close(got, exp, tol)
        assert not bad.any(), (name, dt, z[bad][:3], got[bad][:3], exp[bad][:3])
    if name not in ("expm1", "sign"):
        z = GRID.astype(dt)
        got, exp = device(name, z), expected(name, z)
        bad = ~parts_close(got, exp, 8 * RES[dt])
        assert not bad.any(), (name, dt, z[bad][:4], got[bad][:4], exp[bad][:4])
    # strided and reversed views, out= (test_exp.py:186-212)
    z = (rng.uniform(-2, 2, 72) + 1j * rng.uniform(-2, 2, 72)).astype(dt)
    dz = dp.asarray(z)
    fn = getattr(dp, NAMES.get(name, name))
    for step in (-4, -3, -2, -1, 2, 3, 4):
        assert parts_close(fn(dz[::step]).asnumpy(), expected(name, z[::step]), tol).all()
    out = dp.empty(72, dtype=dt)
    fn(dz, out=out)
    assert parts_close(out.asnumpy(), expected(name, z), tol).all()


@pytest.mark.parametrize("dt", ["c8", "c16"])
def test_expm1_special_values_of_the_reference(dt):
    inf, nan = np.inf, np.nan
    vals = [complex(0.0, 0.0), complex(-0.0, 0.0), complex(1.0, inf), complex(1.0, nan), complex(inf, 0.0),
            complex(-inf, 1.0), complex(inf, 1.0), complex(-inf, inf), complex(inf, inf), complex(-inf, nan),
            complex(inf, nan), complex(nan, 0.0), complex(nan, 1.0), complex(nan, nan)]
    cis_1 = complex(np.cos(1.0), np.sin(1.0))
    c_nan = complex(nan, nan)
    with np.errstate(all="ignore"):
        want = np.asarray([complex(0.0, 0.0), complex(0.0, 0.0), c_nan, c_nan, complex(inf, 0.0), 0.0 * cis_1 - 1.0,
                           inf * cis_1 - 1.0, complex(-1.0, 0.0), complex(inf, nan), complex(-1.0, 0.0),
                           complex(inf, nan), complex(nan, 0.0), c_nan, c_nan], dtype=dt)
    got = device("expm1", np.asarray(vals, dtype=dt))
    assert parts_close(got, want, RES[dt]).all(), (got, want)
    assert not np.signbit(got[:2].real).any()


@pytest.mark.parametrize("dt", ["c8", "c16"])
@pytest.mark.parametrize("name", ["arcsin", "arccos", "arctan", "arcsinh", "arccosh", "arctanh"])
def test_inverse_functions_of_large_arguments(name, dt):
    eps = np.finfo("f8" if dt == "c16" else "f4").eps
    thr1 = 1 / eps
    thr2 = np.sqrt(thr1) / 2
    vals = [complex(-4e7, 1.0), complex(-9e7, 1.0), complex(-1e8, 1.0), complex(-4.45712982e8, 1.0),
            complex(thr1, 1.0), complex(thr2, 1.0), complex(np.nextafter(thr1, np.inf), 1.0),
            complex(np.nextafter(thr2, np.inf), 1.0)]
    for m in (4e7, 9e7, 1e8, 4.45e8):
        vals += [complex(sx * m, sy * m) for sx, sy in itertools.product((1, -1), repeat=2)]
    z = np.array(vals, dtype=dt)
    got, exp = device(name, z), expected(name, z)
    assert not np.isinf(got.real).any() and not np.isinf(got.imag).any()
    assert parts_close(got, exp, 8 * RES[dt]).all(), (got, exp)


@pytest.mark.parametrize("dt", ["c8", "c16"])
def test_division_comparisons_maximum_and_power(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(9)
    sp = [np.nan, np.inf, -np.inf, 0.0, -0.0, 1.0, -1.0, 2.5]
    g = np.array([complex(a, b) for a, b in itertools.product(sp, repeat=2)])
    a, b = (m.ravel().astype(dt) for m in np.meshgrid(g, g))
    da, db = dp.asarray(a), dp.asarray(b)
    with warnings.catch_warnings(), np.errstate(all="ignore"):
        warnings.simplefilter("ignore")
        assert parts_close(dp.divide(da, db).asnumpy(), a / b, 8 * RES[dt]).all()
        # mixed real / complex operands promote to the complex type
        r = rng.uniform(1, 3, a.size).astype("f4" if dt == "c8" else "f8")
        assert parts_close(dp.divide(dp.asarray(r), db).asnumpy(), r / b, 8 * RES[dt]).all()
        assert parts_close(dp.divide(da, dp.asarray(r)).asnumpy(), a / r, 8 * RES[dt]).all()
        assert parts_close((1 / db).asnumpy(), dp.reciprocal(db).asnumpy(), RES[dt]).all()
        clean = ~(np.isnan(a.real) | np.isnan(a.imag) | np.isnan(b.real) | np.isnan(b.imag))
        for name in ("less", "less_equal", "greater", "greater_equal"):
            got = getattr(dp, name)(da, db).asnumpy()
            assert got.dtype == np.bool_
            np.testing.assert_array_equal(got[clean], getattr(np, name)(a, b)[clean])
            # next to a NaN an ordered comparison of unequal real parts is false (less.hpp:60-101)
            nan_im = (np.isnan(a.imag) | np.isnan(b.imag)) & (a.real != b.real)
            assert not got[nan_im].any()
        for name in ("maximum", "minimum"):
            got = getattr(dp, name)(da, db).asnumpy()
            exp = getattr(np, name)(a, b)
            np.testing.assert_array_equal(np.isnan(got.real) | np.isnan(got.imag), np.isnan(exp.real) | np.isnan(exp.imag))
            np.testing.assert_array_equal(got[clean], exp[clean])
        zs = (rng.uniform(-3, 3, 4001) + 1j * rng.uniform(-3, 3, 4001)).astype(dt)
        zt = (rng.uniform(-3, 3, 4001) + 1j * rng.uniform(-3, 3, 4001)).astype(dt)
        # the exponent b log a reaches |.| ~ 15: its rounding shows up as a relative error of the
        # modulus, so the values are compared as complex numbers
        assert modulus_close(dp.power(dp.asarray(zs), dp.asarray(zt)).asnumpy(), np.power(zs, zt), 50 * RES[dt]).all()
        assert modulus_close((dp.asarray(zs) ** 3).asnumpy(), zs ** 3, 50 * RES[dt]).all()


@pytest.mark.parametrize("dt", ["i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8"])
def test_integer_power_by_squaring(dt):
    """pow.hpp:74-95: repeated squaring with wrap-around; a negative exponent gives 0."""
    import dpnp_b200 as dp

    rng = np.random.default_rng(3)
    info = np.iinfo(dt)
    base = rng.integers(max(info.min, -12), min(info.max, 12), 3001, endpoint=True).astype(dt)
    ex = rng.integers(0, 9, 3001).astype(dt)
    got = dp.power(dp.asarray(base), dp.asarray(ex)).asnumpy()
    assert got.dtype == np.dtype(dt)
    with np.errstate(all="ignore"):
        np.testing.assert_array_equal(got, np.power(base, ex))          # NumPy wraps the same way
    if info.min < 0:
        neg = dp.power(dp.asarray(np.array([2, -3, 1, 0], dtype=dt)), dp.asarray(np.array([-1, -2, -5, -1], dtype=dt)))
        np.testing.assert_array_equal(neg.asnumpy(), np.zeros(4, dtype=dt))
    x = dp.arange(10, dtype="i4")                                        # test_pow.py:112-119
    sq = dp.square(x)
    x **= 2
    np.testing.assert_array_equal(x.asnumpy(), sq.asnumpy())
    # the type matrix of test_pow.py:44-77 on ones
    for d2 in ("i1", "u2", "i4", "u8", "f2", "f4", "f8", "c8", "c16"):
        r = dp.power(dp.ones(127, dtype=dt), dp.ones(127, dtype=d2))
        e = np.power(np.ones(1, dtype=dt), np.ones(1, dtype=d2))
        assert r.dtype == e.dtype and (r.asnumpy() == e).all(), (dt, d2)


@pytest.mark.parametrize("dt", ["c8", "c16"])
def test_complex_extremes_and_searches(dt):
    """max / min / argmax / argmin of complex arrays over every axis: the (real, imaginary) order
    with NaN as the extreme (math_utils.hpp:99-131, reductions.hpp:1914-1963) -- NumPy's rule."""
    import dpnp_b200 as dp

    rng = np.random.default_rng(17)
    x = (rng.integers(-3, 4, (37, 53, 5)) + 1j * rng.integers(-3, 4, (37, 53, 5))).astype(dt)   # many ties
    d = dp.asarray(x)
    for ax in (None, 0, 1, 2):
        np.testing.assert_array_equal(dp.max(d, axis=ax).asnumpy(), np.max(x, axis=ax))
        np.testing.assert_array_equal(dp.min(d, axis=ax).asnumpy(), np.min(x, axis=ax))
        np.testing.assert_array_equal(dp.argmax(d, axis=ax).asnumpy(), np.argmax(x, axis=ax))
        np.testing.assert_array_equal(dp.argmin(d, axis=ax).asnumpy(), np.argmin(x, axis=ax))
    big = (rng.normal(0, 1, 300001) + 1j * rng.normal(0, 1, 300001)).astype(dt)
    db = dp.asarray(big)
    assert dp.max(db).asnumpy() == big.max() and int(dp.argmin(db).asnumpy()) == int(big.argmin())
    big[123456] = complex(0.5, np.nan)
    big[200000] = complex(np.nan, 0.0)
    db = dp.asarray(big)
    assert int(dp.argmax(db).asnumpy()) == 123456 and int(dp.argmin(db).asnumpy()) == 123456
    m = dp.max(db).asnumpy()
    assert np.isnan(m.real) or np.isnan(m.imag)
