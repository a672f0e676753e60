// Host-side build of the double-precision erf of the kernels (dpnp_b200/csrc/ew_erf.cuh) for
// comparison with correctly rounded values on a machine without a GPU.  Host code only.
#include "../../dpnp_b200/csrc/ew_erf.cuh"

extern "C" void erf_f64_host(long n, const double *x, double *out)
{
    for (long i = 0; i < n; ++i) out[i] = dpb::erf_f64(x[i]);
}
