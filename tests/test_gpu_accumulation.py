"""cumulative_sum / cumulative_prod / cumulative_logsumexp against NumPy: integer results are
bit-exact, floating results within the tolerance of the sums (the partition differs from a
sequential loop)."""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


SHAPES = [((1,), 0), ((1000,), 0), ((5000,), 0), ((3000000,), 0), ((37, 1025), 1), ((37, 1025), 0),
          ((3, 70000), 1), ((70000, 3), 0), ((600, 40000), 0), ((12, 40, 30), 1), ((12, 40, 30), 2),
          ((2, 1 << 21), 1), ((2000, 513), 1)]


@pytest.mark.parametrize("dt", ["i4", "u1", "i8", "f4", "f8", "?"])
@pytest.mark.parametrize("shape,axis", SHAPES, ids=str)
def test_cumsum(shape, axis, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(sum(shape) + axis)
    x = rng.integers(0, 2, shape).astype(dt) if dt == "?" else (rng.normal(0, 1, shape) * 20).astype(dt) \
        if dt[0] != "u" else rng.integers(0, 200, shape).astype(dt)
    got = dp.cumsum(dev(x), axis=axis)
    ref = np.cumsum(x, axis=axis)
    if dt == "?" or dt[0] in "iu":
        ref = ref.astype("u8" if dt == "u1" else "i8")
        assert got.dtype == ref.dtype
        np.testing.assert_array_equal(got.asnumpy(), ref)
    else:
        assert got.dtype == np.dtype(dt)
        exact = np.cumsum(x.astype(np.longdouble), axis=axis)
        mag = np.cumsum(np.abs(x).astype(np.longdouble), axis=axis)
        tol = 1e-5 if dt == "f4" else 1e-12
        assert np.all(np.abs(got.asnumpy().astype(np.longdouble) - exact) <= tol * mag + 1e-30)


def test_cumprod_and_cumlogsumexp():
    import dpnp_b200 as dp

    rng = np.random.default_rng(9)
    x = rng.integers(1, 3, (50, 40)).astype("i4")
    np.testing.assert_array_equal(dp.cumprod(dev(x), axis=1).asnumpy(), np.cumprod(x, axis=1, dtype="i8"))
    np.testing.assert_array_equal(dp.cumprod(dev(x), axis=0).asnumpy(), np.cumprod(x, axis=0, dtype="i8"))
    f = rng.uniform(0.9, 1.1, (7, 5000))
    np.testing.assert_allclose(dp.cumprod(dev(f), axis=1).asnumpy(), np.cumprod(f, axis=1), rtol=1e-11)
    np.testing.assert_allclose(dp.cumprod(dev(f)).asnumpy(), np.cumprod(f), rtol=1e-10)      # flattened
    for dt, tol in (("f4", 2e-5), ("f8", 1e-12)):
        g = rng.normal(0, 4, (9, 3000)).astype(dt)
        for ax in (0, 1):
            got = dp.cumlogsumexp(dev(g), axis=ax).asnumpy()
            ref = np.logaddexp.accumulate(g.astype(np.longdouble), axis=ax)
            np.testing.assert_allclose(got.astype(np.longdouble), ref, rtol=tol, atol=tol)
    gi = rng.integers(-3, 3, 100).astype("i2")
    r = dp.cumlogsumexp(dev(gi))
    assert r.dtype.kind == "f"
    np.testing.assert_allclose(r.asnumpy(), np.logaddexp.accumulate(gi.astype(r.dtype)), rtol=1e-5)


def test_views_dtype_out_and_include_initial():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(10)
    x = rng.integers(-50, 50, (14, 33, 20)).astype("i4")
    d = dev(x)
    for view in (lambda a: a[::2, ::-1, 1:], lambda a: a.transpose(2, 0, 1), lambda a: a[:, 3:30:3, ::-2]):
        vx, vd = view(x), view(d)
        for ax in (0, 1, 2, -1):
            np.testing.assert_array_equal(dp.cumsum(vd, axis=ax).asnumpy(), np.cumsum(vx, axis=ax))
    np.testing.assert_array_equal(dp.cumsum(d).asnumpy(), np.cumsum(x))                  # flattened
    np.testing.assert_array_equal(dp.cumsum(d, axis=1, dtype="i4").asnumpy(), np.cumsum(x, axis=1, dtype="i4"))
    np.testing.assert_allclose(dp.cumsum(d, axis=1, dtype="f4").asnumpy(), np.cumsum(x, axis=1, dtype="f4"))
    np.testing.assert_array_equal(dp.cumsum(d, axis=2, dtype="i2").asnumpy(), np.cumsum(x, axis=2, dtype="i2"))
    out = dp.empty((14, 33, 20), dtype="i8")
    assert dp.cumsum(d, axis=0, out=out) is out
    np.testing.assert_array_equal(out.asnumpy(), np.cumsum(x, axis=0))
    of = dp.empty((14, 33, 20), dtype="f8")                                              # cast into out
    dp.cumsum(d, axis=0, out=of)
    np.testing.assert_array_equal(of.asnumpy(), np.cumsum(x, axis=0).astype("f8"))
    # in place on the tensor level: out is the input
    y = dev(x.astype("i8")).get_array()
    dp.tensor.cumulative_sum(y, axis=2, out=y)
    np.testing.assert_array_equal(dp.asnumpy(y), np.cumsum(x, axis=2))
    # include_initial: one more element along the axis, starting from the identity
    for ax in (0, 2):
        r = dp.cumulative_sum(d, axis=ax, include_initial=True).asnumpy()
        ref = np.concatenate([np.zeros_like(np.take(x, [0], axis=ax), dtype="i8"), np.cumsum(x, axis=ax)], axis=ax)
        np.testing.assert_array_equal(r, ref)
    r = dp.cumulative_prod(dev(np.array([2.0, 3.0, 4.0])), include_initial=True).asnumpy()
    np.testing.assert_array_equal(r, [1.0, 2.0, 6.0, 24.0])
    # zero-dimensional and empty inputs, errors
    np.testing.assert_array_equal(dp.asnumpy(dp.tensor.cumulative_sum(dev(np.array(5)).get_array())), 5)
    assert dp.cumsum(dp.zeros((3, 0)), axis=1).shape == (3, 0)
    with pytest.raises(ValueError):
        dp.tensor.cumulative_sum(d.get_array())                                          # axis=None needs 1-D
    with pytest.raises(ValueError):
        dp.tensor.cumulative_sum(d.get_array(), axis=0, out=dp.empty((14, 33, 20), dtype="i4").get_array())
    # kernel selection
    big = dp.zeros((4, 1 << 20), dtype="f4")
    dp.cumsum(big, axis=1)
    assert _lib.last_kernel() == "scan_rows_vec"
    dp.cumsum(dp.zeros((64, 1 << 17), dtype="f4"), axis=0)
    assert _lib.last_kernel() == "scan_cols"
    dp.cumsum(dp.zeros((5000, 512), dtype="f4"), axis=1)
    assert _lib.last_kernel() == "scan_rows_vec"
