"""The complex elementary functions (dpnp_b200/csrc/ew_complex.cuh) compiled for the HOST and
compared with NumPy: random arguments, the grid of special values {nan, +-inf, +-0, +-1}^2 that
the reference's tests use (tests/tensor/elementwise/test_exp.py:215-235, test_sqrt.py:129-160),
large arguments around 1/eps (test_hyperbolic.py:226-300, test_trigonometric.py:240-280) and the
reference's own expected values for expm1 (test_expm1.py:97-140).  The kernels compile the same
header for the device; tests/test_gpu_complex.py repeats the comparison there."""

import ctypes as C
import itertools
import os
import shutil
import subprocess
import warnings

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "host_harness", "complex_host.cu")
UNARY = ["exp", "log", "sqrt", "sin", "cos", "tan", "sinh", "cosh", "tanh", "arcsin", "arccos", "arctan",
         "arcsinh", "arccosh", "arctanh", "expm1", "log1p", "log2", "log10", "exp2", "reciprocal", "sign"]
RES = {"c8": 1e-6, "c16": 1e-15}          # finfo(...).resolution, as the reference's tests take it


@pytest.fixture(scope="module")
def lib(tmp_path_factory):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is needed to build the host harness")
    out = str(tmp_path_factory.mktemp("cx") / "libcx_host.so")
    cmd = [nvcc, "-O1", "-std=c++17", "-fmad=false", "--expt-relaxed-constexpr", "-shared", "-Xcompiler", "-fPIC",
           "-Wno-deprecated-gpu-targets", "-x", "cu", SRC, "-o", out]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    assert proc.returncode == 0, proc.stderr
    return C.CDLL(out)


def run_unary(lib, name, x):
    x = np.ascontiguousarray(x)
    out = np.empty_like(x)
    rc = lib.cx_unary(UNARY.index(name), int(x.dtype == np.complex128), C.c_long(x.size),
                      x.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    assert rc == 0
    return out


def run_binary(lib, op, a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    out = np.empty_like(a)
    rc = lib.cx_binary(op, int(a.dtype == np.complex128), C.c_long(a.size), a.ctypes.data_as(C.c_void_p),
                       b.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p))
    assert rc == 0
    return out


def parts_close(got, exp, tol):
    """Real and imaginary parts separately, as assert_allclose(dpt.real(Y), np.real(Ynp)) does in
    the reference's tests: NaNs in the same places, infinities with the same sign, the rest
    within atol = rtol = tol."""
    ok = np.ones(got.shape, bool)
    for p, q in ((got.real, exp.real), (got.imag, exp.imag)):
        ok &= np.isnan(p) == np.isnan(q)
        both = ~np.isnan(p) & ~np.isnan(q)
        inf = both & (np.isinf(p) | np.isinf(q))
        ok[inf] &= (p == q)[inf]
        fin = both & ~inf
        ok[fin] &= (np.abs(p - q) <= tol + tol * np.abs(q))[fin]
    return ok


def modulus_close(got, exp, tol):
    """|got - exp| <= tol + tol |exp| on the complex values, which is what assert_allclose does
    with complex arrays in the reference's tests (NaNs in the same places)."""
    nan_g = np.isnan(got.real) | np.isnan(got.imag)
    nan_e = np.isnan(exp.real) | np.isnan(exp.imag)
    with np.errstate(all="ignore"):
        ok = np.abs(got - exp) <= tol + tol * np.abs(exp)
    return np.where(nan_g | nan_e, nan_g == nan_e, ok | (got == exp))


def expected(name, z):
    with warnings.catch_warnings(), np.errstate(all="ignore"):
        warnings.simplefilter("ignore")
        if name == "reciprocal":
            return np.ones((), z.dtype) / z          # test_reciprocal.py:91-108 compares with 1 / z
        if name == "sign":
            return z / np.abs(z)                     # test_sign.py:61-87
        return getattr(np, name)(z)


SPECIAL = [np.nan, np.inf, -np.inf, 0.0, -0.0, 1.0, -1.0]
GRID = np.array([complex(a, b) for a, b in itertools.product(SPECIAL, repeat=2)])


@pytest.mark.parametrize("dt", ["c8", "c16"])
@pytest.mark.parametrize("name", UNARY)
def test_unary_random_arguments(lib, name, dt):
    rng = np.random.default_rng(UNARY.index(name))
    ranges = [(-9, 9), (-88, 88)] if name in ("exp", "expm1") else [(-9, 9), (-0.5, 0.5), (-1e-3, 1e-3)]
    for lo, hi in ranges:
        z = (rng.uniform(lo, hi, 4000) + 1j * rng.uniform(lo, hi, 4000)).astype(dt)
        got, exp = run_unary(lib, name, z), expected(name, z)
        bad = ~parts_close(got, exp, 8 * RES[dt])
        assert not bad.any(), (name, dt, z[bad][:3], got[bad][:3], exp[bad][:3])


@pytest.mark.parametrize("dt", ["c8", "c16"])
@pytest.mark.parametrize("name", [n for n in UNARY if n not in ("expm1", "sign")])
def test_unary_special_values(lib, name, dt):
    z = GRID.astype(dt)
    got, exp = run_unary(lib, name, z), expected(name, z)
    bad = ~parts_close(got, exp, 8 * RES[dt])
    assert not bad.any(), (name, dt, z[bad][:4], got[bad][:4], exp[bad][:4])


@pytest.mark.parametrize("dt", ["c8", "c16"])
def test_expm1_special_values_of_the_reference(lib, dt):
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
    got = run_unary(lib, "expm1", np.asarray(vals, dtype=dt))
    assert parts_close(got, want, RES[dt]).all(), (got, want)
    assert not np.signbit(got[:2].real).any()


@pytest.mark.parametrize("dt", ["c8", "c16"])
@pytest.mark.parametrize("name", ["arcsin", "arccos", "arctan", "arcsinh", "arccosh", "arctanh", "sqrt", "log"])
def test_large_arguments_in_all_quadrants(lib, name, dt):
    eps = np.finfo("f8" if dt == "c16" else "f4").eps
    thr1 = 1 / eps
    thr2 = np.sqrt(thr1) / 2
    vals = []
    for m in (4e7, 9e7, 1e8, 4.45712982e8, thr1, thr2, np.nextafter(thr1, np.inf), np.nextafter(thr2, np.inf),
              1e30 if dt == "c16" else 1e18):
        for sx, sy in itertools.product((1, -1), repeat=2):
            vals += [complex(sx * m, sy * 1.0), complex(sx * 1.0, sy * m), complex(sx * m, sy * m)]
    z = np.array(vals, dtype=dt)
    got, exp = run_unary(lib, name, z), expected(name, z)
    assert not np.isinf(got.real).any() and not np.isinf(got.imag).any()
    bad = ~parts_close(got, exp, 8 * RES[dt])
    assert not bad.any(), (name, dt, z[bad][:4], got[bad][:4], exp[bad][:4])


def test_acosh_of_zero_with_nan(lib):
    # acosh(+-0 + NaN j) = NaN +- pi/2 j (test_hyperbolic.py:208-222)
    got = run_unary(lib, "arccosh", np.array([complex(0.0, np.nan), complex(-0.0, np.nan)]))
    assert np.isnan(got.real).all() and np.allclose(np.abs(got.imag), np.pi / 2)


@pytest.mark.parametrize("dt", ["c8", "c16"])
def test_division_powers_and_ordering(lib, dt):
    rng = np.random.default_rng(5)
    res = RES[dt]
    sp = SPECIAL + [2.5]
    g = np.array([complex(a, b) for a, b in itertools.product(sp, repeat=2)])
    a, b = (m.ravel().astype(dt) for m in np.meshgrid(g, g))
    with np.errstate(all="ignore"):
        # quotients: every pair of special values agrees with NumPy (4096 pairs)
        assert parts_close(run_binary(lib, 0, a, b), a / b, 8 * res).all()
        za = (rng.uniform(-9, 9, 5000) + 1j * rng.uniform(-9, 9, 5000)).astype(dt)
        zb = (rng.uniform(-9, 9, 5000) + 1j * rng.uniform(-9, 9, 5000)).astype(dt)
        assert parts_close(run_binary(lib, 0, za, zb), za / zb, 4 * res).all()
        big = 1e300 if dt == "c16" else 1e37          # no overflow where the plain formula would
        zc, zd = (za * big).astype(dt), (zb * big).astype(dt)
        assert parts_close(run_binary(lib, 0, zc, zd), zc / zd, 4 * res).all()
        zs = (rng.uniform(-3, 3, 5000) + 1j * rng.uniform(-3, 3, 5000)).astype(dt)
        zt = (rng.uniform(-3, 3, 5000) + 1j * rng.uniform(-3, 3, 5000)).astype(dt)
        assert modulus_close(run_binary(lib, 1, zs, zt), np.power(zs, zt), 50 * res).all()
        ints = np.array([complex(k, 0) for k in rng.integers(-6, 7, 5000)], dtype=dt)
        assert modulus_close(run_binary(lib, 1, zs, ints), np.power(zs, ints), 50 * res).all()
        got = run_binary(lib, 2, a, b)                  # (less, less_equal) in the two parts
        # NumPy orders complex numbers the same way except next to NaNs, where every ordered
        # comparison here is false (utils/math_utils.hpp:43-97 of the reference)
        clean = ~(np.isnan(a.real) | np.isnan(a.imag) | np.isnan(b.real) | np.isnan(b.imag))
        assert np.array_equal((got.real != 0)[clean], (a < b)[clean])
        assert np.array_equal((got.imag != 0)[clean], (a <= b)[clean])
        mixed = ~clean & (a.real != b.real)
        assert not (got.real != 0)[mixed & (np.isnan(a.imag) | np.isnan(b.imag))].any()
