// Host-side build of the complex elementary functions (dpnp_b200/csrc/ew_complex.cuh) so that
// the same source the kernels use can be compared with NumPy on a machine without a GPU.
// Built by tests/test_complex_host.py with nvcc; host code only, no kernel, no device call.
#include "../../dpnp_b200/csrc/ew_complex.cuh"

using namespace dpb;

template <class F> static int unary(int op, long n, const cplx<F> *in, cplx<F> *out)
{
    for (long i = 0; i < n; ++i) {
        const cplx<F> z = in[i];
        cplx<F> r;
        switch (op) {
        case 0: r = cx::c_exp(z); break;
        case 1: r = cx::c_log(z); break;
        case 2: r = cx::c_sqrt(z); break;
        case 3: r = cx::c_sin(z); break;
        case 4: r = cx::c_cos(z); break;
        case 5: r = cx::c_tan(z); break;
        case 6: r = cx::c_sinh(z); break;
        case 7: r = cx::c_cosh(z); break;
        case 8: r = cx::c_tanh(z); break;
        case 9: r = cx::c_asin(z); break;
        case 10: r = cx::c_acos(z); break;
        case 11: r = cx::c_atan(z); break;
        case 12: r = cx::c_asinh(z); break;
        case 13: r = cx::c_acosh(z); break;
        case 14: r = cx::c_atanh(z); break;
        case 15: r = cx::c_expm1(z); break;
        case 16: r = cx::c_log1p(z); break;
        case 17: r = cx::c_log2(z); break;
        case 18: r = cx::c_log10(z); break;
        case 19: r = cx::c_exp2(z); break;
        case 20: r = cx::c_reciprocal(z); break;
        case 21: r = cx::c_sign(z); break;
        default: return 1;
        }
        out[i] = r;
    }
    return 0;
}

template <class F> static int binary(int op, long n, const cplx<F> *a, const cplx<F> *b, cplx<F> *out)
{
    for (long i = 0; i < n; ++i) {
        switch (op) {
        case 0: out[i] = cx::c_div(a[i], b[i]); break;
        case 1: out[i] = cx::c_pow(a[i], b[i]); break;
        case 2: out[i] = cplx<F>(cx::c_less(a[i], b[i]) ? F(1) : F(0), cx::c_less_equal(a[i], b[i]) ? F(1) : F(0)); break;
        default: return 1;
        }
    }
    return 0;
}

extern "C" int cx_unary(int op, int is_double, long n, const void *in, void *out)
{
    return is_double ? unary<double>(op, n, static_cast<const cdouble *>(in), static_cast<cdouble *>(out))
                     : unary<float>(op, n, static_cast<const cfloat *>(in), static_cast<cfloat *>(out));
}

extern "C" int cx_binary(int op, int is_double, long n, const void *a, const void *b, void *out)
{
    return is_double ? binary<double>(op, n, static_cast<const cdouble *>(a), static_cast<const cdouble *>(b),
                                      static_cast<cdouble *>(out))
                     : binary<float>(op, n, static_cast<const cfloat *>(a), static_cast<const cfloat *>(b),
                                     static_cast<cfloat *>(out));
}
