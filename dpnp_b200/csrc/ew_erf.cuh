// erf in double precision with an error below one unit in the last place, and the float /
// float16 variants computed through it.
//
// The reference takes erf from the SYCL device library / oneMKL
// (dpnp/backend/kernels/elementwise_functions/erf.hpp:51-99), accurate to about an ulp.  The CUDA
// math library's erf, measured on B200 against correctly rounded values, reaches 1.32 ulp (1.6 % of
// the arguments in [1/4, 1/2) are off by more than 1 ulp), which would leave no room for "at most
// 2 ulp from the reference", and costs about 55 FP64 instructions per element, above what the FP64
// pipe issues in the time HBM needs for 16 bytes.  So the function is written out here, in about 25
// FP64 instructions and one 32-byte table load:
//
//   |x| < 1/16     erf(x) = x + x * (EFX + z * Q(z)),  z = x^2: the Maclaurin series with the leading
//                  x added last, so that every rounding error before it is scaled by about 0.13
//   1/16..6        r = the multiple of 1/128 nearest to |x| (one addition of 1.5 * 2^45 rounds to it
//                  and leaves the table index in the low mantissa bits), d = |x| - r (exact),
//                  erf(r + d) = E + (e + S d (1 + a1 d + ... + a5 d^5)):  E + e = erf(r) as a
//                  double-double, S = 2/sqrt(pi) exp(-r^2) and r^2 come from the table, and
//                  a_n = (-1)^n H_n(r) / (n+1)! (the Taylor series of erf at r; H_n the Hermite
//                  polynomial) is evaluated from r.  |S d| <= 0.0045 while E >= 0.07, so the rounding
//                  errors of the series reach the result scaled down and the last addition rounds
//                  once.  Truncation: 0.03 ulp at worst.
//   |x| >= 6       the table's last point, erf = 1 (erf(x) rounds to 1 from 5.93 on);  NaN -> NaN
//
// The table and the constants come from gen_erf_tables.py (mpmath, 60 digits).  Fused multiply-adds
// are written explicitly (the library is otherwise compiled without contraction).
#pragma once

#include <math.h>
#include <string.h>

#include "common.cuh"

namespace dpb {

#include "erf_tables.inc"

// 32 bytes per table point: one sector per lookup
#ifdef __CUDACC__
static __device__ __align__(32) const double kErfTableDevice[kErfEntries * 4] = {DPB_ERF_TABLE_VALUES};
#endif
alignas(32) static const double kErfTableHost[kErfEntries * 4] = {DPB_ERF_TABLE_VALUES};

namespace erf_detail {
DPB_HD constexpr double poly(double, double c0) { return c0; }
template <typename... Rest>
DPB_HD double poly(double u, double c_high, double c_next, Rest... rest)
{
    // coefficients from the highest power down: Horner
    return poly(u, fma(c_high, u, c_next), rest...);
}
}  // namespace erf_detail

DPB_HD double erf_f64(double x)
{
    const double ax = fabs(x);
    if (ax < 0.0625) {
        const double z = x * x;
        const double q = DPB_ERF_SMALL_Q(z);
        return fma(x, fma(z, q, kErfEfx), x);
    }
    constexpr double kShift = 0x1.8p45;            // ulp = 1/128
    const double ac = fmin(ax, 6.0);               // drops a NaN, which is put back below
    const double zs = ac + kShift;
    const double r = zs - kShift;
    const double d = ac - r;
#ifdef __CUDA_ARCH__
    const int k = __double2loint(zs);
    // one 32-byte load per lookup (the gathers run at the rate of the L1, which counts accesses)
    double e_hi, e_lo, s, u;
    asm("ld.global.nc.v4.f64 {%0, %1, %2, %3}, [%4];"
        : "=d"(e_hi), "=d"(e_lo), "=d"(s), "=d"(u)
        : "l"(kErfTableDevice + 4 * k));
#else
    unsigned long long bits;
    memcpy(&bits, &zs, sizeof bits);
    const int k = static_cast<int>(bits & 0xffffffffull);
    const double *row = kErfTableHost + 4 * k;
    const double e_hi = row[0], e_lo = row[1], s = row[2], u = row[3];
#endif
    using erf_detail::poly;
    const double a1 = -r;
    const double a2 = poly(u, DPB_ERF_A2);
    const double a3 = r * poly(u, DPB_ERF_A3);
    const double a4 = poly(u, DPB_ERF_A4);
    const double a5 = r * poly(u, DPB_ERF_A5);
    double p = fma(a5, d, a4);
    p = fma(p, d, a3);
    p = fma(p, d, a2);
    p = fma(p, d, a1);
    const double sd = s * d;
    const double c = fma(sd, p * d, sd);
    const double res = e_hi + (e_lo + c);
    return (x != x) ? x + x : copysign(res, x);
}

}  // namespace dpb
