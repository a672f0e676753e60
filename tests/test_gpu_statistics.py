"""var / std / count_nonzero / logsumexp / reduce_hypot against the CPU oracle (NumPy in
extended precision where the value is a floating-point accumulation)."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = {"f4": 2e-5, "f8": 1e-12}


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


@pytest.mark.parametrize("dt", ["f4", "f8", "i4", "u1"])
@pytest.mark.parametrize("shape,axis", [((1000,), None), ((37, 129), 0), ((37, 129), 1), ((5, 6, 70), (0, 2)),
                                        ((4, 300000), 1), ((64, 3, 5), None)])
def test_var_and_std(shape, axis, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(len(shape) * 100 + sum(shape))
    x = (rng.normal(3, 2, shape) * 10).astype(dt)
    d = dev(x)
    res_dt = np.dtype(dt) if dt[0] == "f" else np.dtype("f8")
    xl = x.astype(np.longdouble)
    for ddof in (0, 1):
        for keep in (False, True):
            v = dp.var(d, axis=axis, ddof=ddof, keepdims=keep)
            s = dp.std(d, axis=axis, ddof=ddof, keepdims=keep)
            ev = xl.var(axis=axis, ddof=ddof, keepdims=keep)
            assert v.dtype == res_dt and s.dtype == res_dt and v.shape == np.shape(ev)
            tol = RTOL["f4" if res_dt == np.dtype("f4") else "f8"]
            np.testing.assert_allclose(v.asnumpy().astype(np.longdouble), ev, rtol=tol * 20)
            np.testing.assert_allclose(s.asnumpy().astype(np.longdouble), np.sqrt(ev), rtol=tol * 20)
    # array-API spelling, method-free calls on the tensor level
    np.testing.assert_array_equal(dp.var(d, axis=axis, correction=1).asnumpy(), dp.var(d, axis=axis, ddof=1).asnumpy())


def test_var_edge_cases():
    import dpnp_b200 as dp

    x = dev(np.arange(6.0).reshape(2, 3))
    assert np.all(np.isnan(dp.var(x, axis=1, ddof=3).asnumpy()))          # no degrees of freedom left
    np.testing.assert_array_equal(dp.var(x, axis=()).asnumpy(), np.zeros((2, 3)))
    with pytest.raises(ValueError):
        dp.var(x, ddof=1, correction=1)
    with pytest.raises(TypeError):
        dp.std(x, ddof="1")
    with pytest.raises(ValueError):
        dp.tensor.var(dev(np.ones(3, "c8")).get_array())
    out = dp.empty(2)
    assert dp.std(x, axis=1, out=out) is out
    np.testing.assert_allclose(out.asnumpy(), np.arange(6.0).reshape(2, 3).std(axis=1), rtol=1e-15)
    assert dp.var(x, dtype="f4").dtype == np.dtype("f4")


@pytest.mark.parametrize("dt", ["f4", "f8", "i2", "?"])
def test_count_nonzero(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(3)
    x = rng.integers(0, 3, (40, 50, 6)).astype(dt)
    d = dev(x)
    for axis in (None, 0, 1, 2, (0, 2)):
        got = dp.count_nonzero(d, axis=axis)
        assert got.dtype == np.dtype("i8")
        np.testing.assert_array_equal(got.asnumpy(), np.count_nonzero(x, axis=axis))
    np.testing.assert_array_equal(dp.count_nonzero(d, axis=1, keepdims=True).asnumpy(),
                                  np.count_nonzero(x, axis=1, keepdims=True))


@pytest.mark.parametrize("dt", ["f2", "f4", "f8", "i4"])
def test_logsumexp_and_reduce_hypot(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(4)
    x = (rng.normal(0, 3, (33, 70, 9))).astype(dt)
    d = dev(x)
    res_dt = np.dtype(dt) if dt[0] == "f" else np.dtype("f8")
    tol = {"f2": 4e-3, "f4": 2e-5, "f8": 1e-12}[res_dt.str[1:]]
    xl = x.astype(np.longdouble)
    for axis in (None, 0, 1, 2, (1, 2)):
        lse = dp.logsumexp(d, axis=axis)
        m = xl.max(axis=axis, keepdims=True)
        ref = np.log(np.exp(xl - m).sum(axis=axis)) + np.squeeze(m, axis=axis if axis is not None else None)
        assert lse.dtype == res_dt
        np.testing.assert_allclose(lse.asnumpy().astype(np.longdouble), ref, rtol=tol, atol=tol)
        hyp = dp.reduce_hypot(d, axis=axis)
        assert hyp.dtype == res_dt
        np.testing.assert_allclose(hyp.asnumpy().astype(np.longdouble), np.sqrt((xl * xl).sum(axis=axis)), rtol=tol)
    # identities and special values
    z = dp.zeros((3, 0), dtype="f4")
    assert np.all(dp.logsumexp(z, axis=1).asnumpy() == -np.inf)
    np.testing.assert_array_equal(dp.reduce_hypot(z, axis=1).asnumpy(), np.zeros(3, "f4"))
    s = dev(np.array([[-np.inf, -np.inf], [np.inf, 1.0], [np.nan, 1.0]]))
    got = dp.logsumexp(s, axis=1).asnumpy()
    assert got[0] == -np.inf and got[1] == np.inf and np.isnan(got[2])
    with pytest.raises(ValueError):
        dp.logsumexp(dev(np.ones(3, "c8")))
    assert dp.logsumexp(d, axis=0, dtype="f8").dtype == np.dtype("f8")


# ---- known-answer cases of the reference's own tests
def test_reference_var_std_literals():
    """dpnp/tests/tensor/test_tensor_statistical_functions.py:176-230."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    x = dev(np.arange(9, dtype="f4").reshape(3, 3)).get_array()
    g = lambda r: dp.asnumpy(r)
    np.testing.assert_allclose(g(dpt.var(x)), np.float32(6.666666507720947), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.var(x, correction=3)), np.float32(10.0), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.std(x)), np.sqrt(np.float32(6.666666507720947)), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.std(x, correction=3)), np.sqrt(np.float32(10.0)), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.var(x, axis=0)), np.full(3, 6, "f4"), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.var(x, axis=0, correction=1)), np.full(3, 9, "f4"), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.std(x, axis=0)), np.sqrt(np.full(3, 6, "f4")), rtol=1e-6)
    np.testing.assert_allclose(g(dpt.var(x, axis=1)), np.full(3, 0.6666666865348816, "f4"), rtol=1e-6)
    assert dpt.var(x).dtype == np.dtype("f4") and dpt.var(x).shape == ()


def test_reference_logsumexp_hypot_count_nonzero_cases():
    """dpnp/tests/tensor/test_usm_ndarray_reductions.py:321-436 (logsumexp), :445-470 (reduce_hypot),
    :690-705 (count_nonzero)."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    for dt in ("?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8", "f2", "f4", "f8"):
        m = dp.ones(100, dtype=dt).get_array()
        r = dpt.logsumexp(m)
        assert r.dtype.kind == "f"
        tol = np.finfo(r.dtype).resolution
        # closed form 1 + log(100) (the reference compares with NumPy's sequential reduction in the
        # result type, which for float16 is itself 1.4e-3 away from the exact value)
        np.testing.assert_allclose(float(dp.asnumpy(r)), 1 + np.log(100.0), rtol=tol, atol=tol)
        h = dpt.reduce_hypot(m)
        assert h.dtype.kind == "f"
        np.testing.assert_allclose(float(dp.asnumpy(h)), 10.0, rtol=tol, atol=tol)
    y = dpt.logsumexp(dp.empty((0,), dtype="f4").get_array())
    assert y.shape == () and dp.asnumpy(y) == -np.inf
    y = dpt.reduce_hypot(dp.empty((0,), dtype="f4").get_array())
    assert y.shape == () and dp.asnumpy(y) == 0
    m = dp.ones((3, 4, 5, 6, 7), dtype="f4").get_array()
    s = dpt.logsumexp(m, axis=(1, 2, -1))
    assert s.shape == (3, 6)
    np.testing.assert_allclose(dp.asnumpy(s), np.full((3, 6), np.log(140.0) + 1, "f4"), rtol=1e-6)
    mi = dp.ones((3, 4, 5, 6, 7), dtype="i4").get_array()
    assert dpt.logsumexp(mi, axis=(1, 2, -1), keepdims=True).shape == (3, 1, 1, 6, 1)
    a = dp.ones((10, 0, 10)).get_array()
    assert dpt.logsumexp(a, keepdims=True).shape == (1, 1, 1)
    assert dpt.logsumexp(a, axis=(0, 1), keepdims=True).shape == (1, 1, 10)
    assert dpt.logsumexp(a, axis=(1, 2), keepdims=True).shape == (10, 1, 1)
    assert dpt.logsumexp(a, axis=(0, 2), keepdims=True).shape == (1, 0, 1)
    assert dpt.logsumexp(a[0], keepdims=True).shape == (1, 1)
    assert dpt.logsumexp(dp.ones(()).get_array()).shape == ()
    with pytest.raises(ValueError):
        dpt.logsumexp(dp.zeros(1, dtype="c8").get_array())
    assert dpt.logsumexp(dp.zeros((8, 10), dtype="f4").get_array(), axis=0).shape == (10,)
    for dt in ("?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8", "f2", "f4", "f8", "c8", "c16"):
        x = dp.ones(10, dtype=dt)
        r = dpt.count_nonzero(x.get_array())
        assert int(dp.asnumpy(r)) == 10 and r.dtype == np.dtype("i8")
        x[3:6] = 0
        assert int(dp.asnumpy(dpt.count_nonzero(x.get_array()))) == 7
