// erf in double precision with an error below one unit in the last place, and the float /
// float16 variants computed through it.
//
// The reference takes erf from the SYCL device library / oneMKL
// (dpnp/backend/kernels/elementwise_functions/erf.hpp:51-99), accurate to about an ulp.  The CUDA
// math library's erf, measured on B200 against correctly rounded values, stays below 0.92 ulp for
// |x| >= 1/2 but reaches 1.32 ulp below 1/2 (1.6 % of the arguments in [1/4, 1/2) are off by more
// than 1 ulp), which would leave no room for "at most 2 ulp from the reference".  So the small
// arguments are evaluated here:
//
//   |x| < 1/2      erf(x) = x + x * (EFX + z * Q(z)),  z = x^2: the Maclaurin series with the leading
//                  x added last, so that every rounding error before it is scaled by about 0.13
//                  (measured maximum 0.66 ulp)
//   otherwise      the math library's erf
//
// The coefficients come from gen_erf_tables.py (mpmath, 60 digits).  Fused multiply-adds are written
// explicitly (the library is otherwise compiled without contraction).  A table-driven form that
// covered every argument within 0.67 ulp (44 Taylor intervals up to 6) was measured too: its 13
// gathered loads per call held the elementwise kernel at 0.32 of the HBM roofline, so it was dropped.
#pragma once

#include <math.h>

#include "common.cuh"

namespace dpb {

#include "erf_tables.inc"

DPB_HD double erf_f64(double x)
{
    if (fabs(x) < 0.5) {
        const double z = x * x;
        const double q = DPB_ERF_SMALL_Q(z);
        return fma(x, fma(z, q, kErfEfx), x);
    }
    return erf(x);
}

}  // namespace dpb
