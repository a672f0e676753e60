"""Parity of the reduction engine (CUDA) with the CPU oracle.

Integer sums, max/min and argmax/argmin are bit-exact; floating sums must satisfy
|got - exact| <= tol * sum(|x_i|) with tol = 1e-5 (f32) / 1e-12 (f64) against an
extended-precision oracle (the condition-aware form of the stated relative tolerance:
rows of N(0,1) values may sum to almost zero)."""

import ctypes as C
import zlib

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu

SUM_TOL = {"f4": 1e-5, "f8": 1e-12, "f2": 2e-3}


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


def check_float_sum(got, x, axis, dt):
    exact, mag = orc.sum_exact(x, axis=axis)
    err = np.abs(np.asarray(got, dtype=np.longdouble) - exact)
    bound = SUM_TOL[dt] * np.asarray(mag) + np.finfo(np.dtype(dt)).tiny
    assert np.all(err <= bound), (err.max(), float(np.max(bound)))


SHAPES = [(1,), (1000,), (37, 1025), (1025, 37), (3, 4, 5), (16, 70000), (70000, 16), (300, 300), (2, 3000000),
          (5, 1, 7), (17, 33, 65)]


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("dt", ["f4", "f8", "i4", "u1"])
def test_sum_max_argmax_all_axes(shape, dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(zlib.crc32(repr((shape, dt)).encode()))
    x = (rng.normal(0, 1, shape) * 10).astype(dt) if dt[0] != "u" else rng.integers(0, 200, shape).astype(dt)
    d = dev(x)
    for ax in [None] + list(range(len(shape))):
        s = dp.sum(d, axis=ax).asnumpy()
        if dt[0] == "f":
            assert s.dtype == x.dtype
            check_float_sum(s, x, ax, dt)
        else:
            np.testing.assert_array_equal(s, orc.sum_int(x, axis=ax))
            assert s.dtype == orc.default_accumulation_dtype(x.dtype)
        np.testing.assert_array_equal(dp.max(d, axis=ax).asnumpy(), orc.max_(x, axis=ax))
        np.testing.assert_array_equal(dp.min(d, axis=ax).asnumpy(), orc.min_(x, axis=ax))
        am = dp.argmax(d, axis=ax).asnumpy()
        assert am.dtype == np.int64
        np.testing.assert_array_equal(am, orc.argmax(x, axis=ax))
        np.testing.assert_array_equal(dp.argmin(d, axis=ax).asnumpy(), orc.argmin(x, axis=ax))


@pytest.mark.parametrize("n", [1, 15, 16, 17, 31, 32, 33, 1023, 1024, 1025, 16383, 16385, 65536 + 7])
def test_row_lengths_around_kernel_boundaries(n):
    import dpnp_b200 as dp

    rng = np.random.default_rng(n)
    x = rng.integers(-1000, 1000, (7, n)).astype("i4")
    d = dev(x)
    np.testing.assert_array_equal(dp.sum(d, axis=1).asnumpy(), x.sum(axis=1))
    np.testing.assert_array_equal(dp.sum(d, axis=0).asnumpy(), x.sum(axis=0))
    np.testing.assert_array_equal(dp.argmax(d, axis=1).asnumpy(), x.argmax(axis=1))
    np.testing.assert_array_equal(dp.argmax(d).asnumpy(), x.argmax())
    np.testing.assert_array_equal(dp.sum(d[:, 1:], axis=1).asnumpy(), x[:, 1:].sum(axis=1))   # unaligned rows
    np.testing.assert_array_equal(dp.max(d[:, 1:], axis=0).asnumpy(), x[:, 1:].max(axis=0))


def test_many_ties_resolve_to_the_first_occurrence():
    import dpnp_b200 as dp

    rng = np.random.default_rng(0)
    x = rng.integers(0, 10, (8, 300000)).astype("i4")
    d = dev(x)
    np.testing.assert_array_equal(dp.argmax(d).asnumpy(), x.argmax())
    np.testing.assert_array_equal(dp.argmin(d).asnumpy(), x.argmin())
    np.testing.assert_array_equal(dp.argmax(d, axis=1).asnumpy(), x.argmax(axis=1))
    np.testing.assert_array_equal(dp.argmax(d, axis=0).asnumpy(), x.argmax(axis=0))
    np.testing.assert_array_equal(dp.argmin(d, axis=0).asnumpy(), x.argmin(axis=0))
    c = dev(np.full((3, 100000), 7, dtype="i2"))
    np.testing.assert_array_equal(dp.argmax(c, axis=1).asnumpy(), [0, 0, 0])
    np.testing.assert_array_equal(dp.argmin(c).asnumpy(), 0)
    b = np.zeros(5000, dtype="?")
    b[[1234, 4000]] = True
    np.testing.assert_array_equal(dp.argmax(dev(b)).asnumpy(), 1234)
    np.testing.assert_array_equal(dp.argmin(dev(b)).asnumpy(), 0)


def test_nan_rules():
    import dpnp_b200 as dp

    rng = np.random.default_rng(1)
    for dt in ("f4", "f8", "f2"):
        x = rng.normal(0, 1, (64, 513)).astype(dt)
        x[3, 7] = np.nan
        x[10, 500] = np.nan
        x[10, 20] = np.nan
        x[20, :] = np.inf
        d = dev(x)
        for ax in (None, 0, 1):
            np.testing.assert_array_equal(dp.max(d, axis=ax).asnumpy(), np.max(x, axis=ax))
            np.testing.assert_array_equal(dp.min(d, axis=ax).asnumpy(), np.min(x, axis=ax))
            np.testing.assert_array_equal(dp.argmax(d, axis=ax).asnumpy(), np.argmax(x, axis=ax))
            np.testing.assert_array_equal(dp.argmin(d, axis=ax).asnumpy(), np.argmin(x, axis=ax))
        assert np.isnan(dp.sum(d).asnumpy())


def test_strided_and_permuted_inputs():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(2)
    x = rng.normal(0, 1, (12, 40, 30)).astype("f8")
    d = dev(x)
    views = [(lambda a: a.transpose(2, 0, 1)), (lambda a: a[::2, ::-1, 1::3]), (lambda a: a[:, 5:, :].transpose(1, 2, 0)),
             (lambda a: a[::-1]), (lambda a: a[..., ::2])]
    for v in views:
        vx, vd = v(x), v(d)
        for ax in (None, 0, 1, 2, (0, 2), (1, 2), (0, 1)):
            check_float_sum(dp.sum(vd, axis=ax).asnumpy(), vx, ax, "f8")
            np.testing.assert_array_equal(dp.max(vd, axis=ax).asnumpy(), vx.max(axis=ax))
            if not isinstance(ax, tuple):
                np.testing.assert_array_equal(dp.argmax(vd, axis=ax).asnumpy(), vx.argmax(axis=ax))
    # middle axis of a dense array takes the coalesced outer kernel
    dp.sum(d, axis=1)
    assert _lib.last_kernel().startswith("reduce_outer")
    dp.sum(d, axis=2)
    assert _lib.last_kernel().startswith("reduce_inner")


def test_several_reduction_axes_with_unit_stride_innermost():
    """Reduction over (0, 2) of a C-contiguous array: rows of the inner kernel, one per
    (result, index along axis 0), merged in order by a second pass."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(77)
    for shape, dt in (((9, 40, 300), "f4"), ((3, 5, 40000), "f8"), ((6, 7, 64), "i4"), ((4, 3, 5, 130), "f8")):
        x = (rng.normal(0, 1, shape) * 8).astype(dt)
        x[tuple(s // 2 for s in shape)] = 1000          # a unique maximum
        d = dev(x)
        ax = (0, len(shape) - 1)
        s = dp.sum(d, axis=ax)
        assert _lib.last_kernel().startswith("reduce_inner"), _lib.last_kernel()
        if dt[0] == "f":
            check_float_sum(s.asnumpy(), x, ax, dt)
        else:
            np.testing.assert_array_equal(s.asnumpy(), orc.sum_int(x, axis=ax))
        np.testing.assert_array_equal(dp.max(d, axis=ax).asnumpy(), x.max(axis=ax))
        np.testing.assert_array_equal(dp.min(d, axis=ax).asnumpy(), x.min(axis=ax))
        # flattened search over a view whose rows are not adjacent: (outer index, position) numbering
        v, vx = d[:, 1:, 2:], x[:, 1:, 2:]
        np.testing.assert_array_equal(dp.argmax(v).asnumpy(), vx.argmax())
        np.testing.assert_array_equal(dp.argmin(v).asnumpy(), vx.argmin())
        ties = np.zeros(shape, dt)
        ties[1:, 1:, 2:] = 5                              # first occurrence wins across rows
        np.testing.assert_array_equal(dp.argmax(dev(ties)[:, :, 1:]).asnumpy(), ties[:, :, 1:].argmax())


def test_leading_axis_with_many_columns_gives_each_thread_its_columns():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(78)
    for shape, dt, kernel in (((64, 1 << 19), "f8", "reduce_outer_cols_vec"),
                              ((19, 700003), "f4", "reduce_outer_cols_scalar"),
                              ((3, 33, 1 << 18), "i4", "reduce_outer_cols_vec")):
        x = (rng.normal(0, 1, shape) * 50).astype(dt)
        d = dev(x)
        s = dp.sum(d, axis=0)
        assert _lib.last_kernel() == kernel, _lib.last_kernel()
        if dt[0] == "f":
            check_float_sum(s.asnumpy(), x, 0, dt)
        else:
            np.testing.assert_array_equal(s.asnumpy(), orc.sum_int(x, axis=0))
        np.testing.assert_array_equal(dp.max(d, axis=0).asnumpy(), x.max(axis=0))
        x[::2] = np.round(x[::2] / 25)                  # many ties: first occurrence must win
        d = dev(x)
        np.testing.assert_array_equal(dp.argmax(d, axis=0).asnumpy(), x.argmax(axis=0))
        assert _lib.last_kernel() == kernel
        np.testing.assert_array_equal(dp.argmin(d, axis=0).asnumpy(), x.argmin(axis=0))
        if len(shape) == 3:
            np.testing.assert_array_equal(dp.max(d, axis=1).asnumpy(), x.max(axis=1))
            np.testing.assert_array_equal(dp.argmax(d, axis=1).asnumpy(), x.argmax(axis=1))


def test_keepdims_out_and_dtype():
    import dpnp_b200 as dp

    rng = np.random.default_rng(3)
    x = rng.integers(-50, 50, (6, 7, 8)).astype("i4")
    d = dev(x)
    for ax in (None, 1, (0, 2)):
        r = dp.sum(d, axis=ax, keepdims=True)
        np.testing.assert_array_equal(r.asnumpy(), x.sum(axis=ax, keepdims=True))
        np.testing.assert_array_equal(dp.max(d, axis=ax, keepdims=True).asnumpy(), x.max(axis=ax, keepdims=True))
    np.testing.assert_array_equal(dp.argmax(d, axis=1, keepdims=True).asnumpy(), x.argmax(axis=1, keepdims=True))
    o = dp.empty((6, 8), dtype="i8")
    assert dp.sum(d, axis=1, out=o) is o
    np.testing.assert_array_equal(o.asnumpy(), x.sum(axis=1))
    of = dp.empty((6, 8), dtype="f4")                      # out of another type: cast afterwards
    dp.sum(d, axis=1, out=of)
    np.testing.assert_array_equal(of.asnumpy(), x.sum(axis=1).astype("f4"))
    np.testing.assert_array_equal(dp.sum(d, dtype="f4").asnumpy(), x.sum(dtype="f4"))
    np.testing.assert_array_equal(dp.sum(d, axis=0, dtype="i4").asnumpy(), x.sum(axis=0, dtype="i4"))
    np.testing.assert_array_equal(dp.sum(d, axis=0, dtype="i2").asnumpy(), x.sum(axis=0, dtype="i2"))  # via a cast
    np.testing.assert_array_equal(dp.sum(dev(x.astype("i1")), dtype="?").asnumpy(), True)
    np.testing.assert_array_equal(dp.prod(dev(np.arange(1, 11, dtype="i4"))).asnumpy(), 3628800)
    np.testing.assert_array_equal(d.sum(axis=2).asnumpy(), x.sum(axis=2))
    np.testing.assert_array_equal(d.max().asnumpy(), x.max())
    with pytest.raises(NotImplementedError):
        dp.sum(d, initial=3)
    with pytest.raises(TypeError):
        dp.argmax(d, axis=(0, 1))
    with pytest.raises(ValueError, match="inconsistent"):
        dp.sum(d, axis=1, out=dp.empty((6, 7), dtype="i8"))


def test_empty_and_degenerate():
    import dpnp_b200 as dp

    z = dev(np.zeros((3, 0, 4), dtype="f4"))
    np.testing.assert_array_equal(dp.sum(z, axis=1).asnumpy(), np.zeros((3, 4), "f4"))
    np.testing.assert_array_equal(dp.sum(z).asnumpy(), np.float32(0))
    assert dp.sum(z, axis=0).shape == (0, 4)
    np.testing.assert_array_equal(dp.prod(z, axis=1).asnumpy(), np.ones((3, 4), "f4"))
    with pytest.raises(ValueError, match="zero-size"):
        dp.max(z, axis=1)
    with pytest.raises(ValueError, match="zero-size"):
        dp.argmax(z)
    with np.errstate(all="ignore"):
        assert np.all(np.isnan(dp.mean(z, axis=1).asnumpy()))
    s = dev(np.float64(3.5))
    np.testing.assert_array_equal(dp.sum(s).asnumpy(), 3.5)
    np.testing.assert_array_equal(dp.argmax(s).asnumpy(), 0)
    np.testing.assert_array_equal(dp.max(dev(np.arange(5)), axis=()).asnumpy(), np.arange(5))


def test_mean():
    import dpnp_b200 as dp

    rng = np.random.default_rng(4)
    x = rng.normal(3, 1, (64, 513)).astype("f4")
    d = dev(x)
    for ax in (None, 0, 1):
        got = dp.mean(d, axis=ax).asnumpy()
        assert got.dtype == np.float32
        np.testing.assert_allclose(got, orc.mean(x, axis=ax), rtol=2e-6)
    xi = rng.integers(0, 100, (50, 60)).astype("i4")
    got = dp.mean(dev(xi), axis=0)
    assert got.dtype == np.float64
    np.testing.assert_allclose(got.asnumpy(), xi.mean(axis=0), rtol=1e-14)
    assert dp.mean(dev(xi), dtype="f4").dtype == np.float32
    np.testing.assert_allclose(d.mean(axis=1, keepdims=True).asnumpy(), x.mean(axis=1, keepdims=True), rtol=2e-6)


def test_float_sum_is_deterministic():
    import dpnp_b200 as dp

    d = dp.random.normal(0, 1, (64, 1 << 18), dtype="f4")
    for ax in (None, 0, 1):
        a = dp.sum(d, axis=ax).asnumpy()
        for _ in range(3):
            np.testing.assert_array_equal(dp.sum(d, axis=ax).asnumpy(), a)


def test_accumulation_dtype_matrix():
    import dpnp_b200 as dp

    rng = np.random.default_rng(5)
    for dt in ("?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8"):
        x = rng.integers(0, 2 if dt == "?" else 100, 5000).astype(dt)
        got = dp.sum(dev(x))
        assert got.dtype == orc.default_accumulation_dtype(x.dtype)
        np.testing.assert_array_equal(got.asnumpy(), orc.sum_int(x))
        np.testing.assert_array_equal(dp.max(dev(x)).asnumpy(), x.max())
        np.testing.assert_array_equal(dp.argmax(dev(x)).asnumpy(), x.argmax())
    h = rng.uniform(0, 1, 3000).astype("f2")
    got = dp.sum(dev(h))
    assert got.dtype == np.float16
    check_float_sum(got.asnumpy(), h, None, "f2")
    c = (rng.normal(0, 1, 2000) + 1j * rng.normal(0, 1, 2000)).astype("c8")
    np.testing.assert_allclose(dp.sum(dev(c)).asnumpy(), c.sum(dtype="c16"), rtol=1e-5, atol=1e-4)


def test_kernel_level_abi():
    """Raw-pointer reduction entry points with element offsets."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    lib = _lib.lib
    rng = np.random.default_rng(6)
    rows, cols = 37, 2049
    x = rng.integers(-100, 100, (rows, cols)).astype("i4")
    dx = dp.get_usm_ndarray(dev(x))
    S = dx.sycl_queue.stream
    i4, i8 = _lib.typenum_of("i4"), _lib.typenum_of("i8")
    r1 = dp.get_usm_ndarray(dp.empty(rows + 2, dtype="i8"))
    _lib.check(lib.dpb_reduce_axis1_contig(_lib.REDUCE_OPS["sum"], i4, i8, rows, cols, dx._ptr, 0, r1._ptr, 2, S))
    np.testing.assert_array_equal(dp.asnumpy(r1)[2:], x.sum(axis=1))
    r0 = dp.get_usm_ndarray(dp.empty(cols, dtype="i4"))
    _lib.check(lib.dpb_reduce_axis0_contig(_lib.REDUCE_OPS["max"], i4, i4, cols, rows, dx._ptr, 0, r0._ptr, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(r0), x.max(axis=0))
    a1 = dp.get_usm_ndarray(dp.empty(rows, dtype="i8"))
    _lib.check(lib.dpb_search_axis1_contig(_lib.SEARCH_OPS["argmax"], i4, rows, cols, dx._ptr, 0, a1._ptr, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(a1), x.argmax(axis=1))
    a0 = dp.get_usm_ndarray(dp.empty(cols, dtype="i8"))
    _lib.check(lib.dpb_search_axis0_contig(_lib.SEARCH_OPS["argmin"], i4, cols, rows, dx._ptr, 0, a0._ptr, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(a0), x.argmin(axis=0))
    # strided: reduce the rows of x[:, ::2] -> iteration (rows; src stride cols; dst stride 1), reduction (ceil(cols/2); stride 2)
    half = (cols + 1) // 2
    it = (C.c_int64 * 3)(rows, cols, 1)
    rd = (C.c_int64 * 2)(half, 2)
    rs = dp.get_usm_ndarray(dp.empty(rows, dtype="i8"))
    _lib.check(lib.dpb_reduce_strided(_lib.REDUCE_OPS["sum"], i4, i8, rows, half, dx._ptr, rs._ptr, 1, it, 0, 0, 1, rd, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(rs), x[:, ::2].sum(axis=1))
    _lib.check(lib.dpb_search_strided(_lib.SEARCH_OPS["argmax"], i4, rows, half, dx._ptr, rs._ptr, 1, it, 0, 0, 1, rd, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(rs), x[:, ::2].argmax(axis=1))
    f4 = _lib.typenum_of("f4")
    assert lib.dpb_reduce_axis1_contig(_lib.REDUCE_OPS["sum"], f4, i4, rows, cols, dx._ptr, 0, r1._ptr, 0, S) == _lib.ERR_RUNTIME
    assert "not supported" in _lib.last_error()
