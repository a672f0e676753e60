"""The CPU oracle reproduces every known-answer case lifted from the reference's tests."""

import numpy as np
import pytest

from oracle import dpnp_oracle as orc
from tests._golden import apply_view, axis_of, load_cases

CASES = load_cases()


def oracle_eval(c):
    x = apply_view(c["x"], c["view"], np)
    if c["params"].get("order") == "F":
        x = np.asfortranarray(x)
    op, ax = c["op"], axis_of(c["params"])
    if op == "sum":
        dt = c["params"].get("dtype")
        if x.dtype.kind == "f" and dt is None:
            s, _ = orc.sum_exact(x, axis=ax)
            return np.asarray(s).astype(x.dtype)
        if dt is not None and np.dtype(dt).kind == "f":
            s, _ = orc.sum_exact(x, axis=ax)
            return np.asarray(s).astype(dt)
        return np.asarray(orc.sum_int(x, axis=ax, dtype=dt))
    if op == "max":
        return np.asarray(orc.max_(x, axis=ax, keepdims=c["params"].get("keepdims", False)))
    if op == "min":
        return np.asarray(orc.min_(x, axis=ax, keepdims=c["params"].get("keepdims", False)))
    if op == "where":
        views = c["params"]["views"]
        return np.asarray(orc.where(apply_view(c["cond"], views.get("cond", []), np),
                                    apply_view(x, views.get("x", []), np),
                                    apply_view(c["y"], views.get("y", []), np)))
    if op == "argmax":
        return np.asarray(orc.argmax(x, axis=ax))
    if op == "argmin":
        return np.asarray(orc.argmin(x, axis=ax))
    if op == "mean":
        with np.errstate(all="ignore"):
            return np.asarray(orc.mean(x, axis=ax))
    if op == "add":
        return orc.binary_result("add", x, c["y"])
    if op in ("exp", "erf"):
        return orc.unary_result(op, x)
    raise AssertionError(op)


@pytest.mark.parametrize("c", CASES, ids=[c["name"] for c in CASES])
def test_oracle_matches_known_answer(c):
    got = oracle_eval(c)
    exp = c["expected"]
    assert got.shape == exp.shape
    if c["exact"]:
        np.testing.assert_array_equal(got, exp)
        if exp.dtype.kind == "f":
            ok = ~np.isnan(exp)  # the sign of a NaN carries no meaning
            np.testing.assert_array_equal(np.signbit(got)[ok], np.signbit(exp)[ok])
    else:
        tol = 8 * np.finfo(exp.dtype).resolution  # the tolerance the reference's tests use
        np.testing.assert_allclose(got, exp, rtol=tol, atol=tol)


def test_c_restatement_agrees_with_numpy_oracle():
    import ctypes as C

    rng = np.random.default_rng(3)
    core = orc.core()
    # strided binary through the explicit indexer
    a = rng.uniform(-2, 2, (5, 7, 4)).astype("f4")
    b = rng.uniform(-2, 2, (4, 1, 7)).astype("f4")
    out = np.empty((4, 5, 7), dtype="f4")
    shape = (C.c_int64 * 3)(4, 5, 7)
    sa = (C.c_int64 * 3)(1, 28, 4)      # a.transpose(2, 0, 1)
    sb = (C.c_int64 * 3)(7, 0, 1)       # b broadcast along the middle axis
    so = (C.c_int64 * 3)(35, 7, 1)
    assert core.orc_binary_strided(2, 0, C.c_int64(out.size), 3, shape, sa, sb, so, orc._p(a), orc._p(b),
                                   orc._p(out)) == 0
    np.testing.assert_array_equal(out, a.transpose(2, 0, 1) * b)
    # sums in extended precision
    x = rng.normal(0, 1, (13, 1000)).astype("f4")
    s = np.empty(13)
    sabs = np.empty(13)
    core.orc_sum_axis1_f32(C.c_int64(13), C.c_int64(1000), orc._p(x), orc._p(s), orc._p(sabs))
    ref, refabs = orc.sum_exact(x, axis=1)
    np.testing.assert_allclose(s, ref.astype("f8"), rtol=1e-15)
    np.testing.assert_allclose(sabs, refabs.astype("f8"), rtol=1e-15)
    # argmax with ties and NaN
    xi = rng.integers(0, 5, (6, 500)).astype("i4")
    mx = np.empty(6, dtype="i4")
    arg = np.empty(6, dtype="i8")
    core.orc_max_argmax_axis1_i32(C.c_int64(6), C.c_int64(500), orc._p(xi), orc._p(mx), orc._p(arg))
    np.testing.assert_array_equal(mx, xi.max(axis=1))
    np.testing.assert_array_equal(arg, xi.argmax(axis=1))
    core.orc_max_argmax_axis1_i32_mt(C.c_int64(6), C.c_int64(500), orc._p(xi), orc._p(mx), orc._p(arg))
    np.testing.assert_array_equal(arg, xi.argmax(axis=1))
    xf = rng.normal(0, 1, (6, 500)).astype("f4")
    xf[2, 77] = np.nan
    xf[2, 300] = np.nan
    mf = np.empty(6, dtype="f4")
    core.orc_max_argmax_axis1_f32(C.c_int64(6), C.c_int64(500), orc._p(xf), orc._p(mf), orc._p(arg))
    np.testing.assert_array_equal(mf, xf.max(axis=1))
    np.testing.assert_array_equal(arg, xf.argmax(axis=1))
    # Black-Scholes: C chain (libm) vs NumPy/SciPy chain; +,-,*,/,sqrt are exact, exp/log/erf may
    # differ in the last bits between libm and NumPy/SciPy
    n = 4096
    p, k, t = rng.uniform(10, 50, n), rng.uniform(10, 50, n), rng.uniform(1, 2, n)
    call, put = orc.black_scholes_c(p, k, t, 0.1, 0.2)
    call_t, put_t = orc.black_scholes_c(p, k, t, 0.1, 0.2, threads=True)
    np.testing.assert_array_equal(call, call_t)
    np.testing.assert_array_equal(put, put_t)
    ec, ep = orc.black_scholes_chain(p, k, t, 0.1, 0.2)
    np.testing.assert_allclose(call, ec, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(put, ep, rtol=1e-12, atol=1e-12)


def test_numpy_exp_log_erf_are_within_one_ulp_of_correct_rounding():
    """The floating tolerance (2 ulp against the reference) is checked on the GPU against
    correctly rounded values; here the same yardstick is applied to the host functions the
    oracle uses, which shows the yardstick itself is sound."""
    import scipy.special as sp

    rng = np.random.default_rng(11)
    x = rng.uniform(-5, 5, 300)
    assert orc.ulp_distance(np.exp(x), orc.mp_reference("exp", x)).max() <= 1.0
    xp = rng.uniform(0.01, 100, 300)
    assert orc.ulp_distance(np.log(xp), orc.mp_reference("log", xp)).max() <= 1.0
    assert orc.ulp_distance(sp.erf(x), orc.mp_reference("erf", x)).max() <= 1.5
