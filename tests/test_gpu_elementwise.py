"""Parity of the elementwise engine (CUDA) with the CPU oracle.

Integer ops, comparisons and add/sub/mul/div/sqrt must be bit-exact; exp/log/erf
must lie within 2 ulp of the reference -- checked as <= 1 ulp (f64 exp/log),
<= 2 ulp (erf) from the correctly rounded value, because the reference's own
bits (oneMKL VM) are not available."""

import ctypes as C
import zlib

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu

ALL = ["?", "i1", "u1", "i2", "u2", "i4", "u4", "i8", "u8", "f2", "f4", "f8", "c8", "c16"]
REAL = ALL[:-2]


def rand(rng, dt, shape, lo=-20, hi=20):
    dt = np.dtype(dt)
    if dt.kind == "b":
        return rng.integers(0, 2, shape).astype(dt)
    if dt.kind == "u":
        return rng.integers(0, hi, shape).astype(dt)
    if dt.kind == "i":
        return rng.integers(lo, hi, shape).astype(dt)
    if dt.kind == "c":
        return (rng.uniform(lo, hi, shape) + 1j * rng.uniform(lo, hi, shape)).astype(dt)
    return rng.uniform(lo, hi, shape).astype(dt)


def dev(x):
    import dpnp_b200 as dp

    return dp.asarray(x)


@pytest.mark.parametrize("n", [0, 1, 2, 31, 32, 33, 127, 1023, 1024, 1025, 4095, 4097, 100003, 1 << 20])
def test_add_f32_contiguous_sizes(n):
    import dpnp_b200 as dp

    rng = np.random.default_rng(n)
    a, b = rng.uniform(-1, 1, n).astype("f4"), rng.uniform(-1, 1, n).astype("f4")
    np.testing.assert_array_equal(dp.add(dev(a), dev(b)).asnumpy(), a + b)


@pytest.mark.parametrize("op", ["add", "subtract", "multiply", "divide", "maximum", "minimum", "less",
                                "less_equal", "greater", "greater_equal", "equal", "not_equal",
                                "logical_and", "logical_or"])
@pytest.mark.parametrize("dt", ALL)
def test_binary_dtype_matrix_is_bit_exact(op, dt):
    import dpnp_b200 as dp

    if dt == "?" and op == "subtract":
        pytest.skip("subtract is not defined for bool")
    rng = np.random.default_rng(zlib.crc32(repr((op, dt)).encode()))
    x, y = rand(rng, dt, 3001), rand(rng, dt, 3001, lo=1)
    exp = orc.binary_result(op, x, y)
    got = getattr(dp, op)(dev(x), dev(y)).asnumpy()
    assert got.dtype == exp.dtype
    if op == "multiply" and np.dtype(dt).kind == "c":
        # (ac - bd) + (ad + bc)i: each product and sum rounds on its own here, while the host
        # library may fuse a multiply-add; the two differ by one rounding of a part
        eps = np.finfo(exp.real.dtype).eps
        scale = np.abs(x) * np.abs(y)
        assert np.all(np.abs(got - exp) <= 2 * eps * scale)
    elif op == "divide" and np.dtype(dt).kind == "c":
        # the quotient is scaled by the larger part of the divisor (four roundings per part):
        # within 4 eps of the host result, relative to |x / y|
        eps = np.finfo(exp.real.dtype).eps
        assert np.all(np.abs(got - exp) <= 4 * eps * np.abs(exp))
    else:
        # (integer division promotes to float64 first; the division itself is exact IEEE)
        np.testing.assert_array_equal(got, exp)


def test_mixed_type_promotion_and_scalars():
    import dpnp_b200 as dp

    rng = np.random.default_rng(1)
    for d1 in REAL:
        for d2 in ("i4", "u8", "f4", "f8"):
            x, y = rand(rng, d1, 257), rand(rng, d2, 257, lo=1)
            for op in ("add", "multiply", "less"):
                exp = orc.binary_result(op, x, y)
                got = getattr(dp, op)(dev(x), dev(y)).asnumpy()
                assert got.dtype == exp.dtype, (op, d1, d2)
                np.testing.assert_array_equal(got, exp, err_msg=f"{op} {d1} {d2}")
    x = rand(rng, "f4", 1000)
    np.testing.assert_array_equal((dev(x) * 0.25).asnumpy(), x * np.float32(0.25))
    np.testing.assert_array_equal((1.0 / dev(x)).asnumpy(), np.float32(1.0) / x)
    np.testing.assert_array_equal((dev(x) - 3).asnumpy(), x - np.float32(3))
    xi = rand(rng, "i4", 1000)
    assert (dev(xi) * 2.5).dtype == np.float64
    np.testing.assert_array_equal((dev(xi) * 2.5).asnumpy(), xi * 2.5)
    np.testing.assert_array_equal((dev(xi) / 4).asnumpy(), xi / 4)
    xu = rand(rng, "u1", 100)
    np.testing.assert_array_equal((dev(xu) > -1).asnumpy(), np.ones(100, bool))


def test_int64_uint64_comparisons_do_not_lose_range():
    import dpnp_b200 as dp

    a = np.array([-1, 0, 2**62, -2**63, 5], dtype="i8")
    b = np.array([2**64 - 1, 0, 2**63, 0, 4], dtype="u8")
    for op, pyop in (("less", lambda p, q: p < q), ("greater_equal", lambda p, q: p >= q),
                     ("equal", lambda p, q: p == q)):
        exp = np.array([pyop(int(p), int(q)) for p, q in zip(a, b)])
        np.testing.assert_array_equal(getattr(dp, op)(dev(a), dev(b)).asnumpy(), exp)
        exp_r = np.array([pyop(int(q), int(p)) for p, q in zip(a, b)])
        np.testing.assert_array_equal(getattr(dp, op)(dev(b), dev(a)).asnumpy(), exp_r)


@pytest.mark.parametrize("dt", ["f2", "f4", "f8"])
def test_unary_exact_ops(dt):
    import dpnp_b200 as dp

    rng = np.random.default_rng(2)
    x = rand(rng, dt, 5003, lo=0.01, hi=50)
    for op in ("sqrt", "negative", "abs", "square", "floor", "ceil", "reciprocal", "positive"):
        exp = orc.unary_result(op, x)
        got = getattr(dp, op)(dev(x)).asnumpy()
        assert got.dtype == exp.dtype
        np.testing.assert_array_equal(got, exp, err_msg=op)


def test_exp_log_erf_ulp_error_f64():
    """Distance to the correctly rounded value (mpmath): at most 1 ulp for exp and log, below 1 ulp
    for erf on a dense sweep of [-6, 6], around the switch of its two forms at 1/2 and on the
    arguments the Black-Scholes chain feeds it.  An implementation within 1 ulp of the true value is
    within 2 ulp of any reference that is itself within 1 ulp."""
    import dpnp_b200 as dp

    rng = np.random.default_rng(3)
    x = np.concatenate([rng.uniform(-20, 20, 1500), rng.uniform(-1e-3, 1e-3, 200), rng.uniform(-700, 700, 500),
                        [0.0, 1.0, -1.0, 700.0, -700.0]])
    ulp = orc.ulp_distance(dp.exp(dev(x)).asnumpy(), orc.mp_reference("exp", x))
    assert ulp.max() <= 1.0, ulp.max()
    xp = np.concatenate([rng.uniform(1e-3, 1e3, 1500), rng.uniform(0.9, 1.1, 300), [1.0, 1e-300, 1e300]])
    ulp = orc.ulp_distance(dp.log(dev(xp)).asnumpy(), orc.mp_reference("log", xp))
    assert ulp.max() <= 1.0, ulp.max()
    p, k, t = rng.uniform(10, 50, 3000), rng.uniform(10, 50, 3000), rng.uniform(1, 2, 3000)
    a, b, z = np.log(p / k), t * -0.1, t * 0.08
    w1, w2 = (a - b + 0.25 * z) / np.sqrt(z), (a - b - 0.25 * z) / np.sqrt(z)
    xe = np.concatenate([rng.uniform(-6, 6, 12000), rng.uniform(-0.5, 0.5, 6000), rng.uniform(0.45, 0.55, 2000),
                         -rng.uniform(0.45, 0.55, 2000), w1, w2, [0.0, 1e-10, 5.9, 0.5, -0.5, 1e-300]])
    ulp = orc.ulp_distance(dp.erf(dev(xe)).asnumpy(), orc.mp_reference("erf", xe))
    assert ulp.max() < 1.0, (ulp.max(), xe[ulp.argmax()])


def test_exp_log_erf_f32_against_correctly_rounded_values():
    """float32: exp and erf are evaluated in double precision and rounded once (within 0.51 ulp);
    log is the math library's logf (1 ulp specified, 0.87 measured)."""
    import dpnp_b200 as dp

    rng = np.random.default_rng(4)
    x = np.concatenate([rng.uniform(-10, 10, 3000), rng.uniform(-87, 88, 2000)]).astype("f4")
    cases = (("exp", x, 0.51), ("log", (np.abs(x) + np.float32(1e-3)), 1.0), ("erf", (x / 3), 0.51))
    for op, arg, bound in cases:
        got = getattr(dp, op)(dev(arg)).asnumpy()
        assert got.dtype == np.float32
        ulp = orc.ulp_distance(got, orc.mp_reference(op, arg.astype("f8")))
        assert ulp.max() <= bound, (op, ulp.max())
    # and a large sample against the float64 evaluation on the host (exact to float32 precision)
    big = rng.uniform(-20, 20, 1 << 20).astype("f4")
    for op, arg, bound in (("exp", big, 0.51), ("log", np.abs(big) + np.float32(1e-3), 1.0), ("erf", big / 5, 0.51)):
        ref = orc.unary_result(op, arg.astype("f8"))
        ulp = orc.ulp_distance(getattr(dp, op)(dev(arg)).asnumpy(), ref.astype(np.longdouble))
        assert ulp.max() <= bound, (op, ulp.max())


def test_special_values():
    import dpnp_b200 as dp

    for dt in ("f4", "f8"):
        x = np.array([np.nan, np.inf, -np.inf, 0.0, -0.0], dtype=dt)
        for op in ("exp", "sqrt", "erf", "negative", "abs"):
            with np.errstate(all="ignore"):
                exp = orc.unary_result(op, x)
            got = getattr(dp, op)(dev(x)).asnumpy()
            np.testing.assert_array_equal(got, exp, err_msg=f"{op} {dt}")
            ok = ~np.isnan(exp)
            np.testing.assert_array_equal(np.signbit(got)[ok], np.signbit(exp)[ok], err_msg=f"{op} {dt}")
        with np.errstate(all="ignore"):
            np.testing.assert_array_equal(dp.log(dev(x)).asnumpy(), np.log(x))
            np.testing.assert_array_equal((dev(x) / dev(x[::-1].copy())).asnumpy(), x / x[::-1])
        np.testing.assert_array_equal(dp.maximum(dev(x), dev(x[::-1].copy())).asnumpy(), np.maximum(x, x[::-1]))


def test_strided_broadcast_and_transposed_operands():
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(5)
    a = rand(rng, "f4", (33, 70, 64))
    b = rand(rng, "f4", (64, 1, 70))
    got = dp.multiply(dev(a).transpose(2, 0, 1), dev(b))
    assert _lib.last_kernel().startswith("ew_transpose")
    assert got.flags.c_contiguous and got.shape == (64, 33, 70)
    np.testing.assert_array_equal(got.asnumpy(), a.transpose(2, 0, 1) * b)
    m = rand(rng, "f8", (257, 130))
    r, c = rand(rng, "f8", 130), rand(rng, "f8", (257, 1))
    np.testing.assert_array_equal((dev(m) + dev(r)).asnumpy(), m + r)
    assert _lib.last_kernel().startswith("ew_rows")
    np.testing.assert_array_equal((dev(m) - dev(c)).asnumpy(), m - c)
    np.testing.assert_array_equal((dev(m).T * dev(m).T).asnumpy(), m.T * m.T)
    np.testing.assert_array_equal((dev(m) * dev(np.ascontiguousarray(m.T)).T).asnumpy(), m * m)
    np.testing.assert_array_equal((dev(m)[::2, ::-3] + dev(m)[::-2, ::3]).asnumpy(), m[::2, ::-3] + m[::-2, ::3])
    x4 = rand(rng, "i2", (5, 6, 7, 8))
    v = dev(x4).transpose(3, 1, 0, 2)
    np.testing.assert_array_equal((v + v[::-1]).asnumpy(), x4.transpose(3, 1, 0, 2) + x4.transpose(3, 1, 0, 2)[::-1])
    x = rand(rng, "f4", 10001)
    np.testing.assert_array_equal((dev(x)[1:] + dev(x)[:-1]).asnumpy(), x[1:] + x[:-1])   # unaligned pointers
    np.testing.assert_array_equal((dev(x)[3::2] * dev(x)[:-3:2]).asnumpy(), x[3::2] * x[:-3:2])
    # odd inner lengths around the vector width, with and without row alignment
    for cols in (1, 3, 4, 5, 7, 8, 9, 31, 33, 129):
        p = rand(rng, "f4", (19, cols + 3))
        q = rand(rng, "f4", (cols,))
        np.testing.assert_array_equal((dev(p)[:, 1:cols + 1] + dev(q)).asnumpy(), p[:, 1:cols + 1] + q)
    # many collapsed dimensions
    x6 = rand(rng, "f4", (3, 4, 2, 5, 3, 4))
    w = dev(x6)[:, ::2, :, ::-1, :, ::3]
    np.testing.assert_array_equal((w + w).asnumpy(), 2 * x6[:, ::2, :, ::-1, :, ::3])


def test_rows_that_start_off_the_16_byte_grid():
    """Rows whose first element sits at the same position within a 16-byte group in every
    operand are processed as a few leading elements plus aligned vectors; any other
    combination of starts takes the element-wise path.  Both must give the same bits."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    rng = np.random.default_rng(31)
    for dt, cols in (("f8", 64), ("f4", 72), ("u1", 96), ("i2", 80)):
        a, b = rand(rng, dt, (33, cols)), rand(rng, dt, (33, cols), 1, 20)
        da, db = dev(a), dev(b)
        out = dp.zeros((33, cols), dtype=dt)
        vec = 16 // np.dtype(dt).itemsize
        for lo in range(0, vec + 1):
            for hi in (cols, cols - 1, cols - vec - 1):
                dp.add(da[:, lo:hi], db[:, lo:hi], out=out[:, lo:hi])
                if 0 < lo < vec:
                    assert _lib.last_kernel() == "ew_rows_vec_head", (_lib.last_kernel(), dt, lo, hi)
                np.testing.assert_array_equal(out.asnumpy()[:, lo:hi], a[:, lo:hi] + b[:, lo:hi])
                dp.multiply(da[:, lo:hi], 3, out=out[:, lo:hi])
                np.testing.assert_array_equal(out.asnumpy()[:, lo:hi], a[:, lo:hi] * np.dtype(dt).type(3))
        # starts that differ between the operands: one element at a time
        dp.add(da[:, 1:-1], db[:, 2:], out=out[:, :-2])
        assert _lib.last_kernel() == "ew_rows_scalar"
        np.testing.assert_array_equal(out.asnumpy()[:, :-2], a[:, 1:-1] + b[:, 2:])
        # a row shorter than the leading part, and a flat array that starts off the grid
        dp.add(da[:, 1:2], db[:, 1:2], out=out[:, 1:2])
        np.testing.assert_array_equal(out.asnumpy()[:, 1:2], a[:, 1:2] + b[:, 1:2])
        fa, fb = da.reshape(-1), db.reshape(-1)
        np.testing.assert_array_equal(dp.add(fa[1:], fb[1:], out=fa[1:].copy()).asnumpy(),
                                      a.reshape(-1)[1:] + b.reshape(-1)[1:])
    # mixed element sizes: f64 rows into an f32 result
    x = rng.normal(0, 1, (20, 50))
    o32 = dp.zeros((20, 50), dtype="f4")
    dp.copyto(o32[:, 1:], dev(x)[:, 1:], casting="same_kind")
    np.testing.assert_array_equal(o32.asnumpy()[:, 1:], x[:, 1:].astype("f4"))


def test_output_layout_follows_order_k():
    import dpnp_b200 as dp

    rng = np.random.default_rng(6)
    a = dev(rand(rng, "f4", (6, 7, 8)))
    assert (a + a).strides == a.strides
    at = a.transpose(2, 0, 1)
    assert (at + at).strides == at.strides                    # permuted dense input keeps its layout
    f = dev(np.asfortranarray(rand(rng, "f4", (6, 7))))
    assert (f + f).flags.f_contiguous
    assert (f + dev(rand(rng, "f4", (6, 7)))).flags.c_contiguous   # any C input -> C result
    assert dp.add(f, f, order="C").flags.c_contiguous
    v = a[:, ::-2]
    r = v + v
    assert r.shape == v.shape and r.strides[1] < 0             # reversed in every input -> reversed result
    np.testing.assert_array_equal(r.asnumpy(), 2 * a.asnumpy()[:, ::-2])


def test_where():
    import dpnp_b200 as dp

    rng = np.random.default_rng(7)
    m = rand(rng, "f8", (257, 130))
    r = rand(rng, "f8", 130)
    for cdt in ("?", "i4", "f4", "u1"):
        cond = rand(rng, cdt, (257, 130), lo=-1, hi=2)
        np.testing.assert_array_equal(dp.where(dev(cond), dev(m), dev(r)).asnumpy(), orc.where(cond, m, r))
    np.testing.assert_array_equal(dp.where(dev(m) > 0, dev(m), 0.0).asnumpy(), np.where(m > 0, m, 0.0))
    np.testing.assert_array_equal(dp.where(dev(m) > 0, 1, -1).asnumpy(), np.where(m > 0, 1, -1))
    mi = rand(rng, "i2", (257, 130))
    got = dp.where(dev(m) > 0, dev(mi), dev(m.astype("f4")))
    assert got.dtype == np.float32
    np.testing.assert_array_equal(got.asnumpy(), np.where(m > 0, mi, m.astype("f4")))
    nanarr = np.array([np.nan, np.inf, -np.inf, 1.0])
    np.testing.assert_array_equal(dp.where(dev(np.array([1, 0, 1, 0], "?")), dev(nanarr), dev(-nanarr)).asnumpy(),
                                  np.where([True, False, True, False], nanarr, -nanarr))
    t = dev(m).T[::2]
    np.testing.assert_array_equal(dp.where(t < 0, t, dev(m).T[1::2]).asnumpy(), np.where(m.T[::2] < 0, m.T[::2], m.T[1::2]))
    assert dp.where(dev(np.zeros((0, 3), "?")), dev(np.zeros((0, 3))), 1.0).shape == (0, 3)


def test_out_in_place_and_overlap():
    import dpnp_b200 as dp

    rng = np.random.default_rng(8)
    m, r = rand(rng, "f8", (100, 30)), rand(rng, "f8", 30)
    d = dev(m.copy())
    d += dev(r)
    np.testing.assert_array_equal(d.asnumpy(), m + r)
    d *= 2
    np.testing.assert_array_equal(d.asnumpy(), (m + r) * 2)
    o = dp.empty_like(dev(m))
    res = dp.add(dev(m), 1.5, out=o)
    assert res is o
    np.testing.assert_array_equal(o.asnumpy(), m + 1.5)
    x = dev(np.arange(10, dtype="f4"))
    dp.add(x[:-1], x[1:], out=x[1:])                # partial overlap: computed through a temporary
    e = np.arange(10, dtype="f4")
    e[1:] = e[:-1] + e[1:]
    np.testing.assert_array_equal(x.asnumpy(), e)
    x = dev(np.arange(10, dtype="f4"))
    dp.add(x, x, out=x)                              # same logical tensor: in place
    np.testing.assert_array_equal(x.asnumpy(), 2 * np.arange(10, dtype="f4"))
    x = dev(np.arange(6, dtype="i4"))
    x += x[::-1]
    np.testing.assert_array_equal(x.asnumpy(), np.full(6, 5, dtype="i4"))
    c = dev(np.zeros(5))
    c[:] = dev(np.arange(5.0))
    c[1:3] = 7
    c[3:] = np.array([8.0, 9.0])
    np.testing.assert_array_equal(c.asnumpy(), [0, 7, 7, 8, 9])
    fm = dev(np.asfortranarray(m))
    fm[...] = dev(m)                                  # layout-changing copy
    np.testing.assert_array_equal(fm.asnumpy(), m)
    np.testing.assert_array_equal(dev(m).astype("f4").asnumpy(), m.astype("f4"))
    np.testing.assert_array_equal(dev(m * 10).astype("i2").asnumpy(), (m * 10).astype("i2"))
    np.testing.assert_array_equal(dev(np.array([-1.5, 2.5, 300.0])).astype("u1").asnumpy()[:2], np.array([255, 2], "u1"))
    np.testing.assert_array_equal(dev(np.array([0, 2, 0, -1], "i1")).astype("?").asnumpy(), [False, True, False, True])


def test_error_messages():
    import dpnp_b200 as dp
    import dpnp_b200.tensor as dpt

    a, b = dev(np.ones((10, 10), "i4")), dev(np.ones(3, "i4"))
    with pytest.raises(ValueError, match="could not be broadcast"):
        dp.add(a, b)
    with pytest.raises(ValueError, match="Output array of type"):
        dp.add(a, a, out=dev(np.ones((10, 10), "f4")))
    with pytest.raises(ValueError, match="shape of input and output arrays are inconsistent"):
        dp.add(a, a, out=dev(np.ones((5, 5), "i4")))
    with pytest.raises(TypeError):
        dp.add(a, [1, 2, 3])
    with pytest.raises(TypeError, match="only takes `out` or `dtype`"):
        dp.add(a, a, out=a, dtype="f4")
    with pytest.raises(NotImplementedError):
        dp.add(a, a, where=False)
    with pytest.raises(ValueError, match="not supported for inputs of data type bool"):
        dp.negative(dev(np.ones(3, "?")))
    with pytest.raises(dp.ExecutionPlacementError):
        dpt.add(1, 2)
    # the native dispatcher validates on its own as well
    from dpnp_b200.tensor import _tensor_elementwise_impl as tei

    ua, uf = dp.get_usm_ndarray(a), dp.get_usm_ndarray(dev(np.ones((10, 10), "f4")))
    with pytest.raises(ValueError, match="unexpected elemental data type"):
        tei._add(ua, ua, uf, ua.sycl_queue)
    with pytest.raises(ValueError, match="shapes are not the same"):
        tei._add(ua, ua, dp.get_usm_ndarray(dev(np.ones((10, 9), "i4"))), ua.sycl_queue)
    with pytest.raises(ValueError, match="overlapping segments"):
        x = dp.get_usm_ndarray(dev(np.ones(10, "i4")))
        tei._add(x[:-1], x[:-1], x[1:], x.sycl_queue)


def test_kernel_level_abi_contig_and_strided():
    """The raw-pointer entry points (the reference's kernel function-pointer signatures)."""
    import dpnp_b200 as dp
    from dpnp_b200 import _lib

    lib = _lib.lib
    rng = np.random.default_rng(9)
    n = 50000
    a, b = rand(rng, "f8", n), rand(rng, "f8", n)
    da, db, do = (dp.get_usm_ndarray(v) for v in (dev(a), dev(b), dp.empty(n)))
    S = do.sycl_queue.stream
    f8 = _lib.typenum_of("f8")
    _lib.check(lib.dpb_binary_contig(_lib.BINARY_OPS["multiply"], f8, f8, f8, n - 3, da._ptr, 1, db._ptr, 2,
                                     do._ptr, 3, S))
    got = dp.asnumpy(do)
    np.testing.assert_array_equal(got[3:], a[1:n - 2] * b[2:n - 1])
    # strided: out[i, j] = a[j, i] + b[0, j] on a 100 x 200 space
    ss = (C.c_int64 * 8)(100, 200, 1, 100, 0, 1, 200, 1)
    a2, b2 = rand(rng, "f8", (200, 100)), rand(rng, "f8", (1, 200))
    da2, db2, do2 = (dp.get_usm_ndarray(v) for v in (dev(a2), dev(b2), dp.empty((100, 200))))
    _lib.check(lib.dpb_binary_strided(_lib.BINARY_OPS["add"], f8, f8, f8, 20000, 2, ss, da2._ptr, 0, db2._ptr, 0,
                                      do2._ptr, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(do2), a2.T + b2)
    _lib.check(lib.dpb_unary_contig(_lib.UNARY_OPS["sqrt"], f8, f8, n, da._ptr, 0, do._ptr, 0, S))
    with np.errstate(all="ignore"):
        np.testing.assert_array_equal(dp.asnumpy(do), np.sqrt(a))
    i4 = _lib.typenum_of("i4")
    assert lib.dpb_binary_contig(_lib.BINARY_OPS["add"], f8, f8, i4, n, da._ptr, 0, db._ptr, 0, do._ptr, 0, S) == _lib.ERR_VALUE
    assert lib.dpb_unary_contig(_lib.UNARY_OPS["exp"], i4, i4, n, da._ptr, 0, do._ptr, 0, S) == _lib.ERR_RUNTIME
    # where / copy-cast at the raw level
    cond = rand(rng, "u1", n, lo=0, hi=2)
    dc = dp.get_usm_ndarray(dev(cond))
    _lib.check(lib.dpb_where_contig(_lib.typenum_of("u1"), f8, n, dc._ptr, da._ptr, db._ptr, do._ptr, S))
    np.testing.assert_array_equal(dp.asnumpy(do), np.where(cond != 0, a, b))
    df = dp.get_usm_ndarray(dp.empty(n, dtype="f4"))
    _lib.check(lib.dpb_copy_cast_contig(f8, _lib.typenum_of("f4"), n, da._ptr, 0, df._ptr, 0, S))
    np.testing.assert_array_equal(dp.asnumpy(df), a.astype("f4"))
