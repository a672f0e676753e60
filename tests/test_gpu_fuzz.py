"""Seeded differential test: random operations on random views (slices, reversals, transposes,
broadcast operands, off-grid starts) against the CPU oracle.  Exact operations must agree bit
for bit; floating-point functions within 4 ulp; sums within the tolerance of the sums."""

import zlib

import numpy as np
import pytest

from oracle import dpnp_oracle as orc

pytestmark = pytest.mark.gpu

EXACT_BINARY = ["add", "subtract", "multiply", "maximum", "minimum", "less", "greater_equal", "equal",
                "bitwise_and", "bitwise_xor", "floor_divide", "remainder", "logical_xor"]
EXACT_UNARY = ["negative", "abs", "square", "sign", "floor", "trunc", "round", "isnan"]
FLOAT_UNARY = ["exp", "log1p", "tanh", "atan", "sinh", "cbrt"]


def random_view(rng, x):
    """A random view of x (NumPy array or device array: the same steps work on both)."""
    steps = []
    nd = x.ndim
    if nd >= 2 and rng.random() < 0.4:
        perm = tuple(int(p) for p in rng.permutation(nd))
        steps.append(("T", perm))
    idx = []
    for _ in range(nd):
        r = rng.random()
        if r < 0.35:
            idx.append(slice(None))
        elif r < 0.6:
            idx.append(slice(int(rng.integers(0, 3)), None))
        elif r < 0.8:
            idx.append(slice(None, None, int(rng.choice([2, 3, -1, -2]))))
        else:
            idx.append(slice(int(rng.integers(0, 2)), -1))
    steps.append(("I", tuple(idx)))
    return steps


def apply_view(x, steps):
    for kind, arg in steps:
        x = x.transpose(arg) if kind == "T" else x[arg]
    return x


def make(rng, dt, shape):
    dt = np.dtype(dt)
    if dt.kind == "f":
        return (rng.normal(0, 3, shape)).astype(dt)
    if dt.kind == "u":
        return rng.integers(0, 50, shape).astype(dt)
    return rng.integers(-50, 50, shape).astype(dt)


@pytest.mark.parametrize("seed", range(40))
def test_random_elementwise_and_reductions(seed):
    import dpnp_b200 as dp

    rng = np.random.default_rng(1000 + seed)
    for _ in range(12):
        nd = int(rng.integers(1, 4))
        shape = tuple(int(s) for s in rng.integers(3, [70, 40, 20][:nd][-1] + 3, nd))
        dt = str(rng.choice(["f4", "f8", "i4", "i8", "u1", "i2"]))
        a = make(rng, dt, shape)
        va_steps = random_view(rng, a)
        xa, da = apply_view(a, va_steps), apply_view(dp.asarray(a), va_steps)
        if xa.size == 0:
            continue
        which = rng.random()
        if which < 0.45:
            ops = [o for o in EXACT_BINARY if not (dt[0] == "f" and o.startswith("bitwise"))]
            op = str(rng.choice(ops))
            mode = rng.random()
            if mode < 0.4:                                   # same-shape second operand, own layout
                b = make(rng, dt, xa.shape)
                xb, db = b, dp.asarray(b)
            elif mode < 0.7 and xa.ndim >= 2:                # broadcast along the first axis
                b = make(rng, dt, xa.shape[1:])
                xb, db = b, dp.asarray(b)
            elif mode < 0.85 and xa.ndim >= 2:               # column operand
                b = make(rng, dt, xa.shape[:-1] + (1,))
                xb, db = b, dp.asarray(b)
            else:                                            # Python scalar
                xb = db = 3 if dt[0] != "f" else 1.5
            if op in ("floor_divide", "remainder") and not np.isscalar(xb):
                xb = np.where(xb == 0, 1, xb).astype(dt)
                db = dp.asarray(xb)
            got = getattr(dp, op)(da, db).asnumpy()
            xbn = np.asarray(xb, dtype=dt) if np.isscalar(xb) else xb
            ref = orc.binary_result(op, xa, np.broadcast_to(xbn, np.broadcast_shapes(xa.shape, np.shape(xbn))))
            assert got.dtype == ref.dtype and got.shape == ref.shape, (op, dt, got.dtype, ref.dtype)
            if ref.dtype.kind == "f":
                nan = np.isnan(ref)
                assert np.array_equal(np.isnan(got), nan), (op, dt)
                np.testing.assert_array_equal(got[~nan], ref[~nan], err_msg=f"{op} {dt} {va_steps}")
            else:
                np.testing.assert_array_equal(got, ref, err_msg=f"{op} {dt} {va_steps}")
        elif which < 0.65:
            ops = EXACT_UNARY if dt[0] != "u" else [o for o in EXACT_UNARY if o != "negative"]
            op = str(rng.choice(ops))
            fn = getattr(dp, op)
            got = fn(da).asnumpy()
            ref = orc.unary_result(op, xa)
            assert got.dtype == ref.dtype, (op, dt)
            np.testing.assert_array_equal(got, ref, err_msg=f"{op} {dt} {va_steps}")
        elif which < 0.8 and dt[0] == "f":
            op = str(rng.choice(FLOAT_UNARY))
            got = getattr(dp, op)(da).asnumpy()
            with np.errstate(all="ignore"):
                ref = orc.unary_result(op, xa)
            fin = np.isfinite(ref)
            assert np.array_equal(np.isfinite(got), fin), (op, dt)
            err = np.abs(got[fin].astype("f8") - ref[fin].astype("f8")) / np.spacing(np.abs(ref[fin])).astype("f8")
            assert err.size == 0 or err.max() <= 4, (op, dt, err.max())
        else:
            axis = None if rng.random() < 0.3 else int(rng.integers(0, xa.ndim))
            kind = str(rng.choice(["sum", "max", "argmin", "cumsum", "count_nonzero"]))
            if kind == "sum":
                got = dp.sum(da, axis=axis).asnumpy()
                if dt[0] == "f":
                    exact, mag = orc.sum_exact(xa, axis=axis)
                    tol = 1e-5 if dt == "f4" else 1e-12
                    assert np.all(np.abs(got.astype(np.longdouble) - exact) <= tol * np.asarray(mag) + 1e-30)
                else:
                    np.testing.assert_array_equal(got, orc.sum_int(xa, axis=axis))
            elif kind == "max":
                np.testing.assert_array_equal(dp.max(da, axis=axis).asnumpy(), xa.max(axis=axis))
            elif kind == "argmin":
                np.testing.assert_array_equal(dp.argmin(da, axis=axis).asnumpy(), xa.argmin(axis=axis))
            elif kind == "count_nonzero":
                np.testing.assert_array_equal(dp.count_nonzero(da, axis=axis).asnumpy(),
                                              np.count_nonzero(xa, axis=axis))
            else:
                ax = 0 if axis is None else axis
                got = dp.cumsum(da, axis=ax).asnumpy()
                if dt[0] == "f":
                    exact = np.cumsum(xa.astype(np.longdouble), axis=ax)
                    mag = np.cumsum(np.abs(xa).astype(np.longdouble), axis=ax)
                    tol = 1e-5 if dt == "f4" else 1e-12
                    assert np.all(np.abs(got.astype(np.longdouble) - exact) <= tol * mag + 1e-30)
                else:
                    ref = np.cumsum(xa, axis=ax, dtype="u8" if dt[0] == "u" else "i8")
                    np.testing.assert_array_equal(got, ref)
