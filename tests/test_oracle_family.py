"""The CPU oracle's restatements of floor_divide / remainder / shifts / proj / round pinned
against the literal answers the reference's own tests assert
(dpnp/tests/tensor/elementwise/test_floor_divide.py:80-147, test_remainder.py:80-153,
test_bitwise_left_shift.py:107-117, test_bitwise_right_shift.py, test_round.py:109-123) and the
running-sum closed forms of dpnp/tests/tensor/test_tensor_accumulation.py:68-127,372-438."""

import numpy as np

from oracle import dpnp_oracle as orc


def test_floor_divide_literals():
    assert orc.floor_divide(np.ones(1, "i4"), np.full(1, -2, "i4"))[0] == -1          # gh-1247
    assert orc.floor_divide(np.full(1, -1, "i4"), np.full(1, 2, "i4"))[0] == -1
    for dt in ("i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8"):
        x = np.arange(10, dtype=dt)
        np.testing.assert_array_equal(orc.floor_divide(x, np.zeros_like(x)), np.zeros(10, dt))
    f = lambda a, b: orc.floor_divide(np.array([a], "f4"), np.array([b], "f4"))[0]
    assert np.isnan(f(np.inf, np.inf)) and np.isnan(f(1.0, np.nan))
    assert f(0.0, -1.0) == 0 and np.signbit(f(0.0, -1.0))
    assert f(-1.0, 0.0) == -np.inf and f(np.inf, -1.0) == -np.inf
    r = f(-1.0, np.inf)                                   # the reference asserts -0.0 (NumPy gives -1)
    assert r == 0 and np.signbit(r)


def test_remainder_literals():
    for dt in ("i1", "i2", "i4", "i8"):
        x = np.arange(-5, -1, 1, dtype=dt)
        three = np.full_like(x, 3)
        np.testing.assert_array_equal(orc.remainder(x, three), np.remainder(x, 3))
        np.testing.assert_array_equal(orc.remainder(three, x), np.remainder(3, x))
    for dt in ("i4", "u4"):
        assert orc.remainder(np.ones(1, dt), np.zeros(1, dt))[0] == 0
    lhs = np.asarray([np.nan, np.inf, 0.0, -0.0, -0.0, 1.0, np.inf, -np.inf], "f4")
    rhs = np.asarray([np.nan, np.inf, -0.0, 1.0, 1.0, 0.0, 1.0, -1.0], "f4")
    with np.errstate(all="ignore"):
        np.testing.assert_allclose(orc.remainder(lhs, rhs), np.remainder(lhs, rhs))
    x = np.linspace(-5, 5, 20)
    np.testing.assert_allclose(orc.remainder(x, np.full_like(x, 3)), np.remainder(x, 3), rtol=1e-15, atol=1e-15)


def test_shift_literals():
    for dt in ("i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8"):
        x = np.ones(255, dtype=dt)
        y = np.full(255, 64, dtype=dt)
        assert not orc.shift_left(x, y).any() and not orc.shift_right(x, y).any()
    assert orc.shift_right(np.array([-8], "i4"), np.array([40], "i4"))[0] == -1
    assert orc.shift_left(np.array([1], "i4"), np.array([-1], "i4"))[0] == 0
    np.testing.assert_array_equal(orc.shift_left(np.array([1, 3], "u1"), np.array([7, 1], "u1")), [128, 6])


def test_round_and_proj_literals():
    x = np.array([np.nan, np.inf, -np.inf, 1.5, 2.5, -1.5, -2.5, 0.0, -0.0])
    y = orc.unary_result("round", x)
    np.testing.assert_array_equal(y[1:], [np.inf, -np.inf, 2.0, 2.0, -2.0, -2.0, 0.0, -0.0])
    np.testing.assert_array_equal(np.signbit(y[1:]), np.signbit(x[1:]))
    np.testing.assert_array_equal(orc.unary_result("round", np.arange(5, dtype="i4")), np.arange(5))
    z = np.array([complex(np.inf, -1), complex(2, -np.inf), complex(1, 2)], "c16")
    p = orc.proj(z)
    assert p[0].real == np.inf and p[0].imag == 0 and np.signbit(p[0].imag)
    assert p[1].real == np.inf and np.signbit(p[1].imag) and p[2] == z[2]


def test_running_sum_closed_forms():
    for dt in ("i1", "i2", "i4", "i8"):
        n = 10000
        ar = np.arange(n).astype(dt)
        x = np.repeat(np.array([1, -1], dtype=dt), n)
        np.testing.assert_array_equal(np.cumsum(x, dtype=dt), np.concatenate((1 + ar, ar[::-1])))
    np.testing.assert_array_equal(np.cumprod(np.full(50, 2, "i8")), 2 ** np.arange(1, 51, dtype="i8"))
    n = 128
    k = np.arange(n, dtype="f8")
    closed = -n + k + np.log1p(-np.exp(-k - 1)) - np.log1p(-np.exp(-1.0))
    np.testing.assert_allclose(np.logaddexp.accumulate(np.arange(-n, 0, dtype="f8")), closed, rtol=1e-13)
