// Elementary functions of a complex argument for the elementwise functors.
//
// The reference computes these with the SYCL experimental complex library plus hand-written
// special-value branches per function (dpnp/tensor/libtensor/include/kernels/elementwise_functions/
// exp.hpp:63-133, cos.hpp:65-180, sinh.hpp, tanh.hpp, sqrt.hpp, log.hpp, acos.hpp ...), and its
// tests define correctness as agreement with NumPy on random arguments and on the grid of special
// values {nan, +-inf, +-0, +-1}^2 (tests/tensor/elementwise/test_exp.py:215-235, test_sqrt.py:129-160,
// test_hyperbolic.py, test_trigonometric.py).  NumPy follows C99 Annex G, so that is what is
// restated here: each function states its special values in the comment above it.
//
// Everything is a __host__ __device__ template over the real type (float, double) so that the same
// source can be checked against NumPy on a machine without a GPU.
#pragma once

#include <math.h>

#include "common.cuh"

namespace dpb {
namespace cx {

template <class F> DPB_HD bool fin(F v) { return isfinite(v); }
template <class F> DPB_HD bool nan_(F v) { return v != v; }
template <class F> DPB_HD bool inf_(F v) { return isinf(v); }
template <class F> DPB_HD F qnan() { return F(NAN); }

template <class F> struct limits_;
template <> struct limits_<float> {
    static DPB_HD float exp_big() { return 88.0f; }       // exp overflows a little above
    static DPB_HD float tanh_big() { return 11.0f; }      // |tanh x| == 1 beyond
    static DPB_HD float huge() { return 1.0e19f; }        // sqrt(max)/small factor: squares still finite
    static DPB_HD float tiny() { return 1.0e-19f; }
};
template <> struct limits_<double> {
    static DPB_HD double exp_big() { return 709.0; }
    static DPB_HD double tanh_big() { return 22.0; }
    static DPB_HD double huge() { return 1.0e153; }
    static DPB_HD double tiny() { return 1.0e-153; }
};

// exp(x) * (c, s) for finite x, without overflow of the intermediate when x is just too large
// for exp but the products are not
template <class F> DPB_HD cplx<F> exp_times(F x, F c, F s, F scale)
{
    if (x > limits_<F>::exp_big()) {
        const F h = exp(x * F(0.5));
        return cplx<F>((h * c) * h * scale, (h * s) * h * scale);
    }
    const F e = exp(x) * scale;
    return cplx<F>(e * c, e * s);
}

// ---------------------------------------------------------------- exp
// exp(x + iy) = e^x (cos y + i sin y).  y == 0: (e^x, y) for every x (keeps NaN + i0, +-inf + i0).
// finite x, y inf/NaN: NaN + iNaN.  x = +inf: finite y != 0: inf cis(y); else (+inf, NaN).
// x = -inf: finite y: +0 cis(y); else (0, 0).  x NaN, y != 0: NaN + iNaN.
template <class F> DPB_HD cplx<F> c_exp(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (y == F(0)) return cplx<F>(exp(x), y);
    if (fin(x)) {
        if (!fin(y)) return cplx<F>(qnan<F>(), qnan<F>());
        return exp_times<F>(x, cos(y), sin(y), F(1));
    }
    if (nan_(x)) return cplx<F>(x, qnan<F>());
    if (x > F(0)) {
        if (fin(y)) return cplx<F>(x * cos(y), x * sin(y));
        return cplx<F>(x, qnan<F>());
    }
    if (fin(y)) return cplx<F>(F(0) * cos(y), F(0) * sin(y));
    return cplx<F>(F(0), F(0));
}

// exp2(z) = exp(z ln 2)
template <class F> DPB_HD cplx<F> c_exp2(cplx<F> z)
{
    const F ln2 = F(0.693147180559945309417232121458176568);
    const F x = z.re, y = z.im;
    if (y == F(0)) return cplx<F>(exp2(x), y);
    if (fin(x) && fin(y)) {
        const F t = y * ln2;
        if (x > F(1020) || (sizeof(F) == 4 && x > F(126))) {
            const F h = exp2(x * F(0.5));
            return cplx<F>((h * cos(t)) * h, (h * sin(t)) * h);
        }
        const F e = exp2(x);
        return cplx<F>(e * cos(t), e * sin(t));
    }
    return c_exp(cplx<F>(x * ln2, y * ln2));
}

// ---------------------------------------------------------------- log
// log(z) = log|z| + i atan2(y, x).  hypot and atan2 give every special value of Annex G:
// log(+-0 + i0) = -inf + i(0 or pi), log(x + i inf) = inf + i pi/2, log(inf + iNaN) = inf + iNaN,
// log(NaN + iy) = NaN + iNaN.  Near |z| = 1 the real part comes from log1p to keep its relative
// accuracy; very large / very small moduli are rescaled so that the squares stay in range.
template <class F> DPB_HD F log_abs(F x, F y)
{
    F ax = fabs(x), ay = fabs(y);
    if (!fin(ax) || !fin(ay)) return log(hypot(ax, ay));
    if (ax < ay) {
        const F t = ax;
        ax = ay;
        ay = t;
    }
    if (ax == F(0)) return -F(INFINITY) ;
    if (ax > F(0.5) && ax < F(2) && ay < F(2)) {
        // |z|^2 - 1 = (ax - 1)(ax + 1) + ay^2, exact enough where it matters
        const F d = (ax - F(1)) * (ax + F(1)) + ay * ay;
        if (d > F(-0.5) && d < F(1)) return F(0.5) * log1p(d);
    }
    return log(hypot(ax, ay));
}

template <class F> DPB_HD cplx<F> c_log(cplx<F> z) { return cplx<F>(log_abs(z.re, z.im), atan2(z.im, z.re)); }

template <class F> DPB_HD cplx<F> c_log2(cplx<F> z)
{
    const F inv_ln2 = F(1.442695040888963407359924681001892137);
    const cplx<F> l = c_log(z);
    return cplx<F>(l.re * inv_ln2, l.im * inv_ln2);
}

template <class F> DPB_HD cplx<F> c_log10(cplx<F> z)
{
    const F inv_ln10 = F(0.434294481903251827651128918916605082);
    const cplx<F> l = c_log(z);
    return cplx<F>(l.re * inv_ln10, l.im * inv_ln10);
}

// log1p(z) = log(1 + z): real part 0.5 log1p(2x + x^2 + y^2) while that is accurate
template <class F> DPB_HD cplx<F> c_log1p(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (!fin(x) || !fin(y)) return c_log(cplx<F>(x + F(1), y));
    const F u = x + F(1);
    const F im = atan2(y, u);
    const F ax = fabs(x), ay = fabs(y);
    if (ax < F(0.5) && ay < F(0.5)) {
        // |1+z|^2 - 1 = x (2 + x) + y^2
        return cplx<F>(F(0.5) * log1p(x * (F(2) + x) + y * y), im);
    }
    return cplx<F>(log_abs(u, y), im);
}

// ---------------------------------------------------------------- sqrt
// Principal square root.  (+-0, +-0) -> (+0, y); y = +-inf -> (inf, y) whatever x is; x NaN ->
// NaN + iNaN; x = +inf -> (inf, NaN or +-0); x = -inf -> (NaN or 0, +-inf); finite x, y NaN ->
// NaN + iNaN.  Otherwise t = sqrt((|x| + |z|)/2) and the other part is y / (2t), with the
// argument scaled by 1/4 (result by 2) or by 4 (result by 1/2) when |z| would leave the range.
template <class F> DPB_HD cplx<F> c_sqrt(cplx<F> z)
{
    F x = z.re, y = z.im;
    if (x == F(0) && y == F(0)) return cplx<F>(F(0), y);
    if (inf_(y)) return cplx<F>(F(INFINITY), y);
    if (nan_(x)) return cplx<F>(x, qnan<F>());
    if (inf_(x)) {
        if (x > F(0)) return cplx<F>(x, nan_(y) ? y : copysign(F(0), y));
        return cplx<F>(nan_(y) ? y : F(0), copysign(F(INFINITY), y));
    }
    if (nan_(y)) return cplx<F>(y, y);
    F scale = F(1);
    const F big = limits_<F>::huge() * F(1e-2), small = limits_<F>::tiny() * F(1e2);
    if (fabs(x) >= big || fabs(y) >= big) {
        x *= F(0.25);
        y *= F(0.25);
        scale = F(2);
    }
    else if (fabs(x) < small && fabs(y) < small) {
        x *= F(4);   // exact; keeps hypot away from the subnormal range in most cases
        y *= F(4);
        scale = F(0.5);
    }
    if (x >= F(0)) {
        const F t = sqrt((x + hypot(x, y)) * F(0.5));
        return cplx<F>(t * scale, (y / (F(2) * t)) * scale);
    }
    const F t = sqrt((-x + hypot(x, y)) * F(0.5));
    return cplx<F>((fabs(y) / (F(2) * t)) * scale, copysign(t, y) * scale);
}

// ------------------------------------------------------- sinh, cosh, tanh
// sinh(x + iy) = sinh x cos y + i cosh x sin y.  x == 0, y inf/NaN: (+-0, NaN).  y == 0, x inf/NaN:
// (x, y).  finite x != 0, y inf/NaN: NaN + iNaN.  x inf: finite y: (x cos y, inf sin y); else
// (+inf, NaN).  x NaN, y != 0: NaN + iNaN.
template <class F> DPB_HD cplx<F> c_sinh(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (fin(x) && fin(y)) {
        if (y == F(0)) return cplx<F>(sinh(x), y);
        const F ax = fabs(x);
        if (ax < limits_<F>::tanh_big()) return cplx<F>(sinh(x) * cos(y), cosh(x) * sin(y));
        // sinh x and cosh x are both e^|x| / 2 here
        const cplx<F> e = exp_times<F>(ax, cos(y), sin(y), F(0.5));
        return cplx<F>(copysign(F(1), x) * e.re, e.im);
    }
    if (x == F(0)) return cplx<F>(x, y - y);
    if (y == F(0)) return cplx<F>(x, y);
    if (fin(x)) return cplx<F>(y - y, y - y);
    if (inf_(x)) {
        if (!fin(y)) return cplx<F>(x * x, y - y);
        return cplx<F>(x * cos(y), F(INFINITY) * sin(y));
    }
    return cplx<F>(x, x * (y - y));
}

// cosh(x + iy) = cosh x cos y + i sinh x sin y.  x == 0, y inf/NaN: (NaN, +-0).  y == 0, x inf:
// (inf, +-0); x NaN: (NaN, +-0).  finite x != 0, y inf/NaN: NaN + iNaN.  x inf: finite y:
// (inf cos y, x sin y); else (inf, NaN).  x NaN, y != 0: NaN + iNaN.
template <class F> DPB_HD cplx<F> c_cosh(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (fin(x) && fin(y)) {
        if (y == F(0)) return cplx<F>(cosh(x), x * y);
        const F ax = fabs(x);
        if (ax < limits_<F>::tanh_big()) return cplx<F>(cosh(x) * cos(y), sinh(x) * sin(y));
        const cplx<F> e = exp_times<F>(ax, cos(y), sin(y), F(0.5));
        return cplx<F>(e.re, copysign(F(1), x) * e.im);
    }
    if (x == F(0)) return cplx<F>(y - y, copysign(F(0), x));
    if (y == F(0)) return cplx<F>(x * x, nan_(x) ? y : copysign(F(0), x) * y);
    if (fin(x)) return cplx<F>(y - y, y - y);
    if (inf_(x)) {
        if (!fin(y)) return cplx<F>(x * x, y - y);
        return cplx<F>((x * x) * cos(y), x * sin(y));
    }
    return cplx<F>(x, x * (y - y));
}

// tanh(x + iy).  Finite arguments: with t = tan y, b = 1 + t^2, s = sinh x, r = sqrt(1 + s^2),
// tanh z = (b r s + i t) / (1 + b s^2); for |x| beyond the point where tanh x rounds to 1 the
// result is (+-1, 4 sin y cos y e^{-2|x|}).  x == 0 and y inf/NaN: (x, NaN); other finite x:
// NaN + iNaN.  x = +-inf: (+-1, +-0 with the sign of sin 2y for finite y, else +0).  x NaN:
// (NaN, y == 0 ? y : NaN).
template <class F> DPB_HD cplx<F> c_tanh(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (nan_(x)) return cplx<F>(x, y == F(0) ? y : x * y);
    if (inf_(x)) {
        const F s2 = fin(y) ? sin(y) * cos(y) : F(0);
        return cplx<F>(copysign(F(1), x), copysign(F(0), fin(y) ? s2 : y));
    }
    if (!fin(y)) return cplx<F>(x == F(0) ? x : y - y, y - y);
    if (fabs(x) >= limits_<F>::tanh_big()) {
        const F e = exp(-fabs(x));
        return cplx<F>(copysign(F(1), x), F(4) * sin(y) * cos(y) * e * e);
    }
    const F t = tan(y);
    const F b = F(1) + t * t;
    const F s = sinh(x);
    const F r = sqrt(F(1) + s * s);
    const F d = F(1) + b * s * s;
    return cplx<F>((b * r * s) / d, t / d);
}

// sin z = -i sinh(iz), cos z = cosh(iz), tan z = -i tanh(iz)   (iz = (-y, x))
template <class F> DPB_HD cplx<F> c_sin(cplx<F> z)
{
    const cplx<F> w = c_sinh(cplx<F>(-z.im, z.re));
    // (NaN, +-inf): C99 leaves the sign of the infinity open; + as NumPy gives it
    if (nan_(w.im) && inf_(w.re)) return cplx<F>(w.im, fabs(w.re));
    return cplx<F>(w.im, -w.re);
}
template <class F> DPB_HD cplx<F> c_cos(cplx<F> z) { return c_cosh(cplx<F>(-z.im, z.re)); }
template <class F> DPB_HD cplx<F> c_tan(cplx<F> z)
{
    const cplx<F> w = c_tanh(cplx<F>(-z.im, z.re));
    return cplx<F>(w.im, -w.re);
}

// expm1(z) = e^x cos y - 1 + i e^x sin y, the real part computed as expm1(x) cos y - 2 sin^2(y/2),
// which keeps small results accurate.  Special values as the reference fixes them
// (elementwise_functions/expm1.hpp:84-131 and tests/tensor/elementwise/test_expm1.py:97-140):
// x = +inf: y inf/NaN -> (inf, NaN); y == 0 -> z; else (+-inf, +-inf) with the signs of cos y,
// sin y.  x = -inf: (-1, +-0) with the sign of y (non-finite y) or of sin y.  x NaN: y == 0 -> z,
// else NaN + iNaN.  (+-0, +-0) -> (0, y).
template <class F> DPB_HD cplx<F> c_expm1(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (inf_(x)) {
        if (x > F(0)) {
            if (!fin(y)) return cplx<F>(x, qnan<F>());
            if (y == F(0)) return z;
            return cplx<F>(copysign(x, cos(y)), copysign(x, sin(y)));
        }
        if (!fin(y)) return cplx<F>(F(-1), copysign(F(0), y));
        return cplx<F>(F(-1), copysign(F(0), sin(y)));
    }
    if (nan_(x)) {
        if (y == F(0)) return z;
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    if (x == F(0) && y == F(0)) return cplx<F>(F(0), y);
    if (x > limits_<F>::exp_big()) {
        const cplx<F> e = c_exp(z);
        return cplx<F>(e.re - F(1), e.im);
    }
    const F sh = (y == F(0)) ? y : sin(y * F(0.5));
    const F re = expm1(x) * cos(y) - F(2) * sh * sh;
    const F im = (y == F(0)) ? y : exp(x) * sin(y);
    return cplx<F>(re, im);
}

// ---------------------------------------------- inverse functions
// Built from real functions of the square roots of 1 +- z (W. Kahan, "Branch cuts for complex
// elementary functions", 1987), which avoids the cancellation in z + sqrt(z^2 - 1):
//   acos z  = 2 atan2(Re sqrt(1-z), Re sqrt(1+z)) + i asinh(Im(conj(sqrt(1+z)) sqrt(1-z)))
//   asin z  = atan2(x, Re(sqrt(1-z) sqrt(1+z)))   + i asinh(Im(conj(sqrt(1-z)) sqrt(1+z)))
//   acosh z = asinh(Re(conj(sqrt(z-1)) sqrt(z+1))) + 2i atan2(Im sqrt(z-1), Re sqrt(z+1))
// For arguments so large that 1 +- z == -+z in the working precision (and for infinities and
// NaNs) the asymptotic forms log(2z) etc. are used, which is also what keeps the results finite
// for |z| around 1/eps.
template <class F> DPB_HD bool any_nan(cplx<F> z) { return nan_(z.re) || nan_(z.im); }

template <class F> DPB_HD cplx<F> c_acosh(cplx<F> z);

template <class F> DPB_HD cplx<F> c_acos(cplx<F> z)
{
    const F x = z.re, y = z.im;
    const F pi = F(3.141592653589793238462643383279502884);
    if (any_nan(z)) {
        // (+-inf, NaN) -> (NaN, -inf); (NaN, +-inf) -> (NaN, -+inf); (+-0, NaN) -> (pi/2, NaN)
        if (inf_(x)) return cplx<F>(y, -F(INFINITY));
        if (inf_(y)) return cplx<F>(x + x, -y);
        if (x == F(0)) return cplx<F>(pi / F(2), y + y);
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    const F big = limits_<F>::huge() * F(1e-3);
    if (fabs(x) > big || fabs(y) > big) {
        // acos z ~ -i log(2z) on the right branch: angle from atan2, size from log|z| + ln 2
        const F ln2 = F(0.693147180559945309417232121458176568);
        const F re = atan2(fabs(y), x);
        F im;
        if (inf_(x) || inf_(y)) im = F(INFINITY);
        else im = log_abs(x * F(0.5), y * F(0.5)) + F(2) * ln2;
        return cplx<F>(re, signbit(y) ? im : -im);
    }
    const cplx<F> a = c_sqrt(cplx<F>(F(1) - x, -y));   // sqrt(1 - z)
    const cplx<F> b = c_sqrt(cplx<F>(F(1) + x, y));    // sqrt(1 + z)
    const F re = F(2) * atan2(a.re, b.re);
    const F im = asinh(b.re * a.im - b.im * a.re);
    return cplx<F>(re, im);
}

template <class F> DPB_HD cplx<F> c_asinh(cplx<F> z);

template <class F> DPB_HD cplx<F> c_asin(cplx<F> z)
{
    // (+-0, NaN) -> z; an infinite part next to a NaN -> (NaN, +-inf with the sign of y); other NaN
    // -> NaN + iNaN
    if (any_nan(z)) {
        if (z.re == F(0)) return z;
        if (inf_(z.re) || inf_(z.im)) return cplx<F>(qnan<F>(), copysign(F(INFINITY), z.im));
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    // asin z = -i asinh(iz)
    const cplx<F> w = c_asinh(cplx<F>(-z.im, z.re));
    return cplx<F>(w.im, -w.re);
}

// asinh(x + iy): odd and conjugate symmetric.  (x, inf) -> (inf, pi/2); (inf, y) -> (inf, 0) for
// finite y; (inf, inf) -> (inf, pi/4); (inf, NaN) -> (inf, NaN); (NaN, 0) -> (NaN, 0);
// (NaN, +-inf) -> (+inf, NaN); other NaN -> NaN + iNaN.
template <class F> DPB_HD cplx<F> c_asinh(cplx<F> z)
{
    const F x = z.re, y = z.im;
    if (any_nan(z)) {
        if (inf_(x)) return cplx<F>(x, y + y);
        if (inf_(y)) return cplx<F>(F(INFINITY), x + x);
        if (y == F(0)) return cplx<F>(x + x, y);
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    const F big = limits_<F>::huge() * F(1e-3);
    if (fabs(x) > big || fabs(y) > big) {
        // asinh z ~ sign(x) (log(2|z|) + i atan2(y, |x|))
        const F ln2 = F(0.693147180559945309417232121458176568);
        F re;
        if (inf_(x) || inf_(y)) re = F(INFINITY);
        else re = log_abs(x * F(0.5), y * F(0.5)) + F(2) * ln2;
        const F im = atan2(y, fabs(x));
        return cplx<F>(copysign(re, x), im);
    }
    // with w = iz: asinh z = -i asin(w); Kahan's asin on w = (-y, x)
    const F wx = -y, wy = x;
    const cplx<F> a = c_sqrt(cplx<F>(F(1) - wx, -wy));   // sqrt(1 - w)
    const cplx<F> b = c_sqrt(cplx<F>(F(1) + wx, wy));    // sqrt(1 + w)
    const F as_re = atan2(wx, a.re * b.re - a.im * b.im);
    const F as_im = asinh(a.re * b.im - a.im * b.re);
    // -i (as_re + i as_im) = as_im - i as_re
    return cplx<F>(as_im, -as_re);
}

// acosh z = +-i acos z, the sign chosen so that the real part is non-negative:
// (NaN handling follows acos; acosh(+-0 + iNaN) = NaN +- i pi/2)
template <class F> DPB_HD cplx<F> c_acosh(cplx<F> z)
{
    const cplx<F> w = c_acos(z);
    if (nan_(w.re) && nan_(w.im)) return w;
    if (nan_(w.re)) return cplx<F>(fabs(w.im), w.re);        // acos gave (NaN, +-inf): acosh = (inf, NaN)
    if (nan_(w.im)) return cplx<F>(w.im, w.re);              // acos gave (pi/2, NaN): acosh = (NaN, pi/2)
    // i w = (-w.im, w.re) when Im z >= 0 (w.im <= 0), else -i w = (w.im, -w.re)
    if (signbit(z.im)) return cplx<F>(fabs(w.im), -w.re);
    return cplx<F>(fabs(w.im), w.re);
}

// atanh(x + iy), odd and conjugate symmetric.  For x >= 0:
//   real = log1p(4x / ((1 - x)^2 + y^2)) / 4,  imag = atan2(2y, (1 - x)(1 + x) - y^2) / 2.
// atanh(1 + i0) = inf + i0; (x, inf) -> (0, pi/2); (inf, y) -> (0, pi/2); (inf, NaN) -> (0, NaN);
// (NaN, inf) -> (+-0, pi/2); (0, NaN) -> (0, NaN); other NaN -> NaN + iNaN.
template <class F> DPB_HD cplx<F> c_atanh(cplx<F> z)
{
    const F x = z.re, y = z.im;
    const F pi_2 = F(1.570796326794896619231321691639751442);
    if (any_nan(z)) {
        if (inf_(x)) return cplx<F>(copysign(F(0), x), y + y);
        if (inf_(y)) return cplx<F>(copysign(F(0), x), copysign(pi_2, y));
        if (x == F(0)) return cplx<F>(x, y + y);
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    if (inf_(x) || inf_(y)) return cplx<F>(copysign(F(0), x), copysign(pi_2, y));
    const F ax = fabs(x), ay = fabs(y);
    if (y == F(0) && ax == F(1)) return cplx<F>(copysign(F(INFINITY), x), y);
    const F big = limits_<F>::huge() * F(1e-3);
    F re, im;
    if (ax > big || ay > big) {
        // atanh z ~ 1/z +- i pi/2:  Re(1/z) = x / |z|^2 without overflow
        const F m = ax > ay ? ax : ay;
        const F sx = ax / m, sy = ay / m;
        re = (sx / (sx * sx + sy * sy)) / m;
        im = pi_2;
    }
    else {
        const F d = (F(1) - ax) * (F(1) - ax) + ay * ay;
        re = F(0.25) * log1p(F(4) * ax / d);
        im = F(0.5) * atan2(F(2) * ay, (F(1) - ax) * (F(1) + ax) - ay * ay);
    }
    return cplx<F>(copysign(re, x), copysign(im, y));
}

template <class F> DPB_HD cplx<F> c_atan(cplx<F> z)
{
    // atan z = -i atanh(iz)
    const cplx<F> w = c_atanh(cplx<F>(-z.im, z.re));
    return cplx<F>(w.im, -w.re);
}

// ---------------------------------------------------------------- arithmetic helpers
// Quotient (a + ib) / (c + id) by scaling with the larger of |c|, |d| (R. L. Smith's method),
// which neither overflows nor underflows where the straightforward formula would; infinities and
// zeros in the divisor follow from IEEE arithmetic on the scaled terms the way NumPy's loops
// (which use the same method) produce them.
template <class F> DPB_HD cplx<F> c_div(cplx<F> n, cplx<F> d)
{
    const F c = d.re, e = d.im;
    const F ac = fabs(c), ae = fabs(e);
    if (ac >= ae) {
        if (ac == F(0) && ae == F(0)) return cplx<F>(n.re / ac, n.im / ac);   // division by zero
        const F r = e / c;
        const F s = F(1) / (c + e * r);
        return cplx<F>((n.re + n.im * r) * s, (n.im - n.re * r) * s);
    }
    const F r = c / e;
    const F s = F(1) / (c * r + e);
    return cplx<F>((n.re * r + n.im) * s, (n.im * r - n.re) * s);
}

template <class F> DPB_HD cplx<F> c_mul(cplx<F> a, cplx<F> b)
{
    return cplx<F>(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
}

template <class F> DPB_HD cplx<F> c_reciprocal(cplx<F> z) { return c_div(cplx<F>(F(1), F(0)), z); }

// z / |z| with |z| = hypot(x, y); 0 for z == 0 (sign.hpp:88-97 of the reference)
template <class F> DPB_HD cplx<F> c_sign(cplx<F> z)
{
    if (z.re == F(0) && z.im == F(0)) return cplx<F>(F(0), F(0));
    const F m = hypot(z.re, z.im);
    return cplx<F>(z.re / m, z.im / m);
}

// Integer powers by repeated squaring, everything else through exp(b log a).
// a^0 = 1 (also for a == 0 and NaN, as NumPy), 0^b = 0 for Re b > 0.
template <class F> DPB_HD cplx<F> c_pow(cplx<F> a, cplx<F> b)
{
    if (b.re == F(0) && b.im == F(0)) return cplx<F>(F(1), F(0));
    if (a.re == F(0) && a.im == F(0)) {
        if (b.re > F(0) && b.im == F(0)) return cplx<F>(F(0), F(0));
        return cplx<F>(qnan<F>(), qnan<F>());
    }
    if (b.im == F(0) && b.re == floor(b.re) && fabs(b.re) <= F(100)) {
        int n = static_cast<int>(b.re);
        const bool neg = n < 0;
        if (neg) n = -n;
        cplx<F> r(F(1), F(0)), p = a;
        while (n) {
            if (n & 1) r = c_mul(r, p);
            n >>= 1;
            if (n) p = c_mul(p, p);
        }
        return neg ? c_reciprocal(r) : r;
    }
    const cplx<F> l = c_log(a);
    return c_exp(c_mul(b, l));
}

// Ordering of complex numbers: real parts decide unless equal, then imaginary parts; a NaN
// anywhere makes every ordered comparison false (utils/math_utils.hpp:43-97 of the reference).
template <class F> DPB_HD bool c_less(cplx<F> a, cplx<F> b)
{
    return (a.re == b.re) ? (a.im < b.im) : (a.re < b.re && !nan_(a.im) && !nan_(b.im));
}
template <class F> DPB_HD bool c_less_equal(cplx<F> a, cplx<F> b)
{
    return (a.re == b.re) ? (a.im <= b.im) : (a.re < b.re && !nan_(a.im) && !nan_(b.im));
}

}  // namespace cx
}  // namespace dpb
