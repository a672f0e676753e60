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


# ---- the known-answer cases of the reference's own tests
# (dpnp/tests/tensor/test_tensor_accumulation.py); expected values are the closed forms the
# tests assert, never the operation under test.
REF = "dpnp/tests/tensor/test_tensor_accumulation.py"


@pytest.mark.parametrize("dt", ["i1", "i2", "i4", "i8"])
def test_reference_cumsum_of_plus_and_minus_ones(dt):
    """:68-127 -- contiguous, strided, reversed, along axis 0 of a matrix and of a strided view;
    the result type is the (possibly wrapping) input type."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    n = 10000
    ar = np.arange(n).astype(dt)
    expected = np.concatenate((1 + ar, ar[::-1]))
    x = dev(np.repeat(np.array([1, -1], dtype=dt), n)).get_array()
    np.testing.assert_array_equal(dp.asnumpy(dpt.cumulative_sum(x, dtype=dt)), expected)
    x = dev(np.repeat(np.array([1, -1], dtype=dt), 2 * n)).get_array()[1::2]
    np.testing.assert_array_equal(dp.asnumpy(dpt.cumulative_sum(x, dtype=dt)), expected)
    x2 = dev(np.repeat(np.array([-1, 1], dtype=dt), 2 * n)).get_array()[-1::-2]
    np.testing.assert_array_equal(dp.asnumpy(dpt.cumulative_sum(x2, dtype=dt)), expected)
    n0, n1 = 1000, 173
    ar = np.arange(n0).astype(dt)
    expected = np.concatenate((1 + ar, ar[::-1]))[:, None]
    m = np.tile(np.repeat(np.array([1, -1], dtype=dt), n0)[:, None], (1, n1))
    r = dp.asnumpy(dpt.cumulative_sum(dev(m).get_array(), dtype=dt, axis=0))
    assert np.all(r == expected)
    m2 = np.tile(np.repeat(np.array([1, -1], dtype=dt), 2 * n0)[:, None], (1, n1))
    r = dp.asnumpy(dpt.cumulative_sum(dev(m2).get_array()[1::2, ::-1], dtype=dt, axis=0))
    assert np.all(r == expected)


def test_reference_scalar_identity_and_basic_cases():
    """:129-173 (scalar input, include_initial identities), :372-404 (cumprod, logcumsumexp),
    :417-428 (closed form of a geometric series), :430-438 (gh-1901), :443-451 (gh-2017)."""
    import dpnp_b200 as dp

    dpt = dp.tensor
    s = dev(np.asarray(1, dtype="i8")).get_array()
    r = dpt.cumulative_sum(s)
    assert r.ndim == 0 and int(dp.asnumpy(r)) == 1
    np.testing.assert_array_equal(dp.asnumpy(dpt.cumulative_sum(s, include_initial=True)), [0, 1])
    x = dp.ones((3, 5), dtype="i4").get_array()
    assert np.all(dp.asnumpy(dpt.cumulative_sum(x, axis=0, include_initial=True))[0, :] == 0)
    assert np.all(dp.asnumpy(dpt.cumulative_sum(x, axis=1, include_initial=True))[:, 0] == 0)
    r = dpt.cumulative_sum(dp.ones(5, dtype="i4").get_array(), include_initial=True)
    assert r.shape == (6,) and dp.asnumpy(r)[0] == 0
    assert dp.asnumpy(dpt.cumulative_prod(dp.zeros(5, dtype="i4").get_array(), include_initial=True))[0] == 1
    assert dp.asnumpy(dpt.cumulative_logsumexp(dp.ones(5, dtype="f4").get_array(), include_initial=True))[0] == -np.inf

    r = dpt.cumulative_prod(dp.full(50, 2, dtype="i8").get_array())
    np.testing.assert_array_equal(dp.asnumpy(r), 2 ** np.arange(1, 51, dtype="i8"))
    r = dpt.cumulative_prod(dev(np.tile(np.array([2, 0.5], dtype="f4"), 10000)).get_array())
    np.testing.assert_array_equal(dp.asnumpy(r), np.tile(np.array([2, 1], dtype="f4"), 10000))
    r = dpt.cumulative_logsumexp(dp.ones(1000, dtype="f4").get_array())
    tol = 4 * np.finfo("f4").resolution
    np.testing.assert_allclose(dp.asnumpy(r), 1 + np.log(np.arange(1, 1001, dtype="f4")), atol=tol, rtol=tol)
    for fpdt in ("f2", "f4", "f8"):
        n = 128
        k = np.arange(n, dtype="f8")
        closed = -n + k + np.log1p(-np.exp(-k - 1)) - np.log1p(-np.exp(-1.0))
        r = dpt.cumulative_logsumexp(dev(np.arange(-n, 0).astype(fpdt)).get_array())
        tol = 4 * np.finfo(fpdt).eps
        np.testing.assert_allclose(dp.asnumpy(r).astype("f8"), closed, atol=tol * 40, rtol=tol)
    for p in (257, 260, 273, 280, 509, 512):
        n = p * p
        r = dpt.cumulative_sum(dp.ones(n, dtype="i4").get_array(), dtype="i4")
        np.testing.assert_array_equal(dp.asnumpy(r), np.arange(1, n + 1, dtype="i4"))
    for dt in ("i1", "i2", "i4", "i8", "f2", "f4", "f8"):
        r = dpt.cumulative_sum(dev(np.array([-1, 1], dtype=dt)).get_array(), dtype="?")
        assert r.dtype == np.dtype("?") and np.all(dp.asnumpy(r))


def test_reference_nan_propagation_and_type_matrix():
    """:314-349 (NaN stays from its position on), :198-237 (default and requested result types)."""
    import dpnp_b200 as dp
    from dpnp_b200.tensor._type_utils import _default_accumulation_dtype

    dpt = dp.tensor
    for fn in (dpt.cumulative_sum, dpt.cumulative_prod, dpt.cumulative_logsumexp):
        x = np.ones(10, dtype="f4")
        x[4] = np.nan
        r = dp.asnumpy(fn(dev(x).get_array()))
        assert np.all(np.isnan(r[4:])) and not np.any(np.isnan(r[:4]))
    for arg in ("?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8", "f2", "f4", "f8"):
        m = dp.ones(100, dtype=arg).get_array()
        r = dpt.cumulative_sum(m)
        assert r.dtype == _default_accumulation_dtype(np.dtype(arg))
        if arg != "?":
            np.testing.assert_array_equal(dp.asnumpy(r), np.arange(1, 101).astype(r.dtype))
        for out in ("i4", "u8", "f4", "f8"):
            r = dpt.cumulative_sum(m, dtype=out)
            assert r.dtype == np.dtype(out)
            np.testing.assert_array_equal(dp.asnumpy(r), np.arange(1, 101).astype(out))


def test_complex_running_sums_and_products():
    import dpnp_b200 as dp

    rng = np.random.default_rng(21)
    for dt, tol in (("c8", 2e-5), ("c16", 1e-12)):
        x = (rng.normal(0, 1, (6, 3000)) + 1j * rng.normal(0, 1, (6, 3000))).astype(dt)
        for ax in (0, 1):
            got = dp.cumsum(dev(x), axis=ax)
            assert got.dtype == np.dtype(dt)
            ref = np.cumsum(x.astype("c16"), axis=ax)
            mag = np.cumsum(np.abs(x).astype("f8"), axis=ax)
            assert np.all(np.abs(got.asnumpy() - ref) <= tol * mag + 1e-30)
        u = np.exp(1j * rng.uniform(0, 6.28, 200)).astype(dt)          # unit modulus: products stay bounded
        np.testing.assert_allclose(dp.cumprod(dev(u)).asnumpy(), np.cumprod(u.astype("c16")), rtol=tol * 300, atol=tol * 300)


LONG_ROWS = [((1 << 22,), "f4"), ((3, 1 << 20), "f4"), ((1, 5_000_001), "f4"), ((2, 33 * 4096 + 7), "f4"),
             ((1 << 21,), "f8"), ((2, 700_001), "i4"), ((1 << 20,), "c8"), ((67_108_869,), "f8")]


@pytest.mark.parametrize("shape,dt", LONG_ROWS, ids=str)
def test_long_rows_single_pass_its_repair_path_and_the_three_launch_scan(shape, dt):
    """A few long rows are scanned in one pass (tiles chained through published totals).  With
    `scan_lookback_polls` = 0 every wait that is not satisfied at once gives up, so the repair launches
    redo those tiles: the result must have the same bits.  The three-launch scan (-1) partitions the
    sums differently: equal for integers, within the tolerance of the sums for floats."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    def tune(v):
        _lib.check(_lib.lib.dpb_set_tuning(b"scan_lookback_polls", v))

    rng = np.random.default_rng(len(shape) + shape[-1])
    if dt == "c8":
        x = (rng.normal(0, 1, shape) + 1j * rng.normal(0, 1, shape)).astype(dt)
    elif dt == "i4":
        x = rng.integers(-1000, 1000, shape).astype(dt)
    else:
        x = rng.normal(0, 1, shape).astype(dt)
    d = dev(x)
    try:
        tune(1 << 20)
        one = dp.cumsum(d, axis=-1)
        assert _lib.last_kernel().startswith("scan_lookback"), _lib.last_kernel()
        one = one.asnumpy()
        tune(0)
        repaired = dp.cumsum(d, axis=-1).asnumpy()
        np.testing.assert_array_equal(repaired, one)
        inplace = dp.asarray(x)
        dp.cumsum(inplace, axis=-1, out=inplace)                       # failed tiles must not have written
        np.testing.assert_array_equal(inplace.asnumpy(), one)
        if len(shape) == 2 and shape[-1] < 3_000_000:
            # the leading identity of include_initial shifts every store by one element (no vector stores)
            tune(1 << 20)
            got = dp.cumulative_sum(d, axis=-1, include_initial=True).asnumpy()
            np.testing.assert_array_equal(got[..., 1:], one)
            assert (got[..., 0] == 0).all()
        tune(-1)
        three = dp.cumsum(d, axis=-1)
        assert _lib.last_kernel().startswith("scan_rows"), _lib.last_kernel()
        three = three.asnumpy()
    finally:
        tune(-1)
    if dt == "i4":
        ref = np.cumsum(x, axis=-1, dtype="i8")
        np.testing.assert_array_equal(one, ref)
        np.testing.assert_array_equal(three, ref)
    else:
        wide = {"f4": "f8", "f8": np.longdouble, "c8": "c16"}[dt]
        exact = np.cumsum(x.astype(wide), axis=-1)
        mag = np.cumsum(np.abs(x).astype("f8"), axis=-1)
        tol = 1e-12 if dt == "f8" else 1e-5
        assert (np.abs(one - exact) <= tol * mag + 1e-30).all()
        assert (np.abs(three - exact) <= tol * mag + 1e-30).all()
