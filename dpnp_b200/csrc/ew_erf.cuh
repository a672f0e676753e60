// erf in double precision with an error below one unit in the last place, and the float /
// float16 variants computed through it.
//
// The reference takes erf from the SYCL device library / oneMKL
// (dpnp/backend/kernels/elementwise_functions/erf.hpp:51-99), whose results are accurate to
// about an ulp; the CUDA math library's erf is specified to 2 ulp, which would leave no room
// for "at most 2 ulp from the reference".  So the function is written out here:
//
//   |x| < 1/2      erf(x) = x + x * (EFX + z * Q(z)),  z = x^2  (Maclaurin series; the leading x
//                  is added last, so everything before it is scaled by ~0.13)
//   1/2..6         intervals of width 1/8 around centres c_i: with t = |x| - c_i (exact),
//                  erf = E_i + (e_i + t * P_i(t)), E_i + e_i = erf(c_i) in double-double and P_i
//                  the Taylor series at c_i; |t * P_i| <= 0.07, so its rounding errors reach the
//                  result scaled down and the last addition rounds once
//   |x| >= 6       +-1;  NaN -> NaN
//
// The tables come from gen_erf_tables.py (mpmath, 60 digits).  Fused multiply-adds are written
// explicitly (the library is otherwise compiled without contraction).
#pragma once

#include <math.h>

#include "common.cuh"

namespace dpb {

#include "erf_tables.inc"

DPB_HD double erf_f64(double x)
{
    const double ax = fabs(x);
    if (!(ax < 6.0)) {
        if (x != x) return x + x;
        return copysign(1.0, x);
    }
    if (ax < 0.5) {
        const double z = x * x;
        const double q = DPB_ERF_SMALL_Q(z);
        return fma(x, fma(z, q, kErfEfx), x);
    }
    int i = static_cast<int>((ax - 0.5) * 8.0);
    if (i > kErfIntervals - 1) i = kErfIntervals - 1;
#ifdef __CUDA_ARCH__
    const double *row = kErfTableDevice + i * kErfRow;
#else
    const double *row = kErfTableHost + i * kErfRow;
#endif
    const double t = ax - (0.5625 + 0.125 * i);
    double p = row[kErfRow - 1];
#pragma unroll
    for (int k = kErfRow - 2; k >= 2; --k) p = fma(p, t, row[k]);
    const double r = row[0] + fma(t, p, row[1]);
    return copysign(r, x);
}

}  // namespace dpb
