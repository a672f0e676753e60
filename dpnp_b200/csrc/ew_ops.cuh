// Elementwise operation functors.  Each functor template takes the argument
// element type(s) and exposes
//   R      - result element type, or NoType when the combination has no kernel
//   apply  - the scalar operation
// The supported type maps follow the *OutputType tables of the reference
// (dpnp/tensor/libtensor/include/kernels/elementwise_functions/<op>.hpp).
#pragma once

#include <math.h>

#include "common.cuh"
#include "ew_complex.cuh"

namespace dpb {

// defined in ew_erf.cuh, which the translation units that instantiate ErfOp include (its table
// and its long body stay out of all the others)
DPB_HD double erf_f64(double x);

struct NoType {};

// arithmetic is carried out in float for half and in the type itself otherwise
template <class T> struct compute_type { using type = T; };
template <> struct compute_type<half_t> { using type = float; };
template <class T> using compute_t = typename compute_type<T>::type;

template <class T> DPB_D compute_t<T> up(T v)
{
    if constexpr (is_half_v<T>) return __half2float(v);
    else return v;
}
template <class T> DPB_D T down(compute_t<T> v)
{
    if constexpr (is_half_v<T>) return __float2half(v);
    else return v;
}

template <class T> DPB_D bool is_nan(T v)
{
    if constexpr (is_half_v<T>) return __hisnan(v);
    else if constexpr (std::is_floating_point_v<T>) return v != v;
    else if constexpr (is_cplx_v<T>) return v.re != v.re || v.im != v.im;
    else return false;
}

// ------------------------------------------------------------------- unary

template <class T> struct NegativeOp {
    using R = std::conditional_t<is_bool_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return T(-x.re, -x.im);
        else if constexpr (is_half_v<T>) return __hneg(x);
        else if constexpr (is_uint_v<T>) return static_cast<T>(T(0) - x);
        else return static_cast<T>(-x);
    }
};

template <class T> struct PositiveOp {
    using R = std::conditional_t<is_bool_v<T>, NoType, T>;
    static DPB_D R apply(T x) { return x; }
};

template <class T> struct real_of { using type = T; };
template <class T> struct real_of<cplx<T>> { using type = T; };
template <class T> using real_of_t = typename real_of<T>::type;

template <class T> struct AbsOp {
    using R = real_of_t<T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return hypot(x.re, x.im);
        else if constexpr (is_half_v<T>) return __habs(x);
        else if constexpr (is_bool_v<T> || is_uint_v<T>) return x;
        else if constexpr (std::is_floating_point_v<T>) return fabs(x);
        else return static_cast<T>(x < 0 ? -x : x);
    }
};

// floating and complex arguments; float16 is computed in float32
#define DPB_FP_UNARY(NAME, FN_F, FN_D, FN_C)                                     \
    template <class T> struct NAME {                                             \
        using R = std::conditional_t<is_fp_v<T> || is_cplx_v<T>, T, NoType>;     \
        static DPB_D R apply(T x)                                                \
        {                                                                        \
            if constexpr (is_cplx_v<T>) return cx::FN_C(x);                      \
            else if constexpr (std::is_same_v<T, double>) return FN_D(x);        \
            else if constexpr (std::is_same_v<T, float>) return FN_F(x);         \
            else return __float2half(FN_F(__half2float(x)));                     \
        }                                                                        \
    };

// float32 exp is evaluated in double and rounded once: the CUDA expf is specified to 2 ulp (1.86
// measured), which would leave no room for "within 2 ulp of the reference"
DPB_D float exp_f32(float x) { return static_cast<float>(exp(static_cast<double>(x))); }
DPB_FP_UNARY(ExpOp, exp_f32, exp, c_exp)      // exp.hpp:63-133
DPB_FP_UNARY(LogOp, logf, log, c_log)         // log.hpp:60-84
DPB_FP_UNARY(SqrtOp, sqrtf, sqrt, c_sqrt)     // sqrt.hpp:62-84
DPB_FP_UNARY(SinOp, sinf, sin, c_sin)         // sin.hpp
DPB_FP_UNARY(CosOp, cosf, cos, c_cos)         // cos.hpp:65-180
DPB_FP_UNARY(TanhOp, tanhf, tanh, c_tanh)     // tanh.hpp
DPB_FP_UNARY(Expm1Op, expm1f, expm1, c_expm1) // expm1.hpp:78-141
DPB_FP_UNARY(Log1pOp, log1pf, log1p, c_log1p) // log1p.hpp
#undef DPB_FP_UNARY

template <class T> struct ReciprocalOp {
    using R = std::conditional_t<is_fp_v<T> || is_cplx_v<T>, T, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return cx::c_reciprocal(x);
        else if constexpr (is_half_v<T>) return __float2half(1.0f / __half2float(x));
        else return T(1) / x;
    }
};

// erf: float16 input is promoted to float32
// (dpnp/backend/extensions/ufunc/elementwise_functions/erf_funcs.cpp:73-85)
// The function itself is erf_f64 of ew_erf.cuh (error below 1 ulp); float arguments go through
// it in double precision and are rounded once.
template <class T> struct ErfOp {
    // every call gathers from a table: fewer elements per thread keep more warps resident to
    // hide the lookups
    static constexpr int kUnroll = 4;
    using R = std::conditional_t<is_half_v<T>, float, std::conditional_t<is_fp_v<T>, T, NoType>>;
    static DPB_D R apply(T x)
    {
        if constexpr (std::is_same_v<T, double>) return erf_f64(x);
        else if constexpr (std::is_same_v<T, float>) return static_cast<float>(erf_f64(static_cast<double>(x)));
        else return static_cast<float>(erf_f64(static_cast<double>(__half2float(x))));
    }
};

template <class T> struct SquareOp {
    using R = std::conditional_t<is_bool_v<T>, int8_t, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_bool_v<T>) return x.v ? int8_t(1) : int8_t(0);
        else if constexpr (is_cplx_v<T>) return T(x.re * x.re - x.im * x.im, x.re * x.im + x.im * x.re);
        else if constexpr (is_half_v<T>) return __hmul(x, x);
        else return static_cast<T>(x * x);
    }
};

template <class T> struct FloorOp {
    using R = std::conditional_t<is_cplx_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_half_v<T>) return hfloor(x);
        else if constexpr (std::is_floating_point_v<T>) return floor(x);
        else return x;
    }
};

template <class T> struct CeilOp {
    using R = std::conditional_t<is_cplx_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_half_v<T>) return hceil(x);
        else if constexpr (std::is_floating_point_v<T>) return ceil(x);
        else return x;
    }
};

template <class T> struct SignOp {
    using R = std::conditional_t<is_bool_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return cx::c_sign(x);
        else if constexpr (is_uint_v<T>) return static_cast<T>(x > 0 ? 1 : 0);
        else if constexpr (is_sint_v<T>) return static_cast<T>((x > 0) - (x < 0));
        else {
            auto v = up(x);
            if (v != v) return x;
            return down<T>(static_cast<compute_t<T>>((v > 0) - (v < 0)));
        }
    }
};

template <class T> struct LogicalNotOp {
    using R = bool_t;
    static DPB_D R apply(T x) { return bool_t(!static_cast<bool>(convert<bool_t>(x))); }
};

template <class T> struct IsNanOp {
    using R = bool_t;
    static DPB_D R apply(T x) { return bool_t(is_nan(x)); }
};

template <class T> DPB_D bool is_inf_scalar(T v)
{
    if constexpr (is_half_v<T>) return __hisinf(v) != 0;
    else if constexpr (std::is_floating_point_v<T>) return isinf(v);
    else return false;
}

template <class T> struct IsInfOp {
    using R = bool_t;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return bool_t(is_inf_scalar(x.re) || is_inf_scalar(x.im));
        else return bool_t(is_inf_scalar(x));
    }
};

template <class T> struct IsFiniteOp {
    using R = bool_t;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>)
            return bool_t(!(is_nan(x) || is_inf_scalar(x.re) || is_inf_scalar(x.im)));
        else return bool_t(!(is_nan(x) || is_inf_scalar(x)));
    }
};

// ------------------------------------------------------------------ binary
// Arithmetic ops are defined for identical argument types only; the Python
// layer promotes the operands first (dpnp/tensor/_type_utils.py:218-251).

template <class A, class B> struct AddOp {
    using R = std::conditional_t<std::is_same_v<A, B>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_bool_v<A>) return bool_t(a.v || b.v);
        else if constexpr (is_cplx_v<A>) return A(a.re + b.re, a.im + b.im);
        else if constexpr (is_half_v<A>) return __hadd(a, b);
        else return static_cast<A>(a + b);
    }
};

template <class A, class B> struct SubtractOp {
    using R = std::conditional_t<std::is_same_v<A, B> && !is_bool_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_cplx_v<A>) return A(a.re - b.re, a.im - b.im);
        else if constexpr (is_half_v<A>) return __hsub(a, b);
        else return static_cast<A>(a - b);
    }
};

template <class A, class B> struct MultiplyOp {
    using R = std::conditional_t<std::is_same_v<A, B>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_bool_v<A>) return bool_t(a.v && b.v);
        else if constexpr (is_cplx_v<A>)
            return A(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
        else if constexpr (is_half_v<A>) return __hmul(a, b);
        else return static_cast<A>(a * b);
    }
};

// true_divide: floating and complex types (integers are promoted to the default
// floating type by the caller, dpnp/tensor/_type_utils.py:89-107).
template <class A, class B> struct TrueDivideOp {
    using R = std::conditional_t<std::is_same_v<A, B> && (is_fp_v<A> || is_cplx_v<A>), A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        // complex quotients (true_divide.hpp:62-113; a real operand next to a complex one is
        // promoted by the caller, which gives the same value as the mixed kernels of the reference)
        if constexpr (is_cplx_v<A>) return cx::c_div(a, b);
        else if constexpr (is_half_v<A>) return __float2half(__half2float(a) / __half2float(b));
        else return a / b;
    }
};

// maximum / minimum propagate NaN (first NaN operand wins).
// Complex operands: the first one wins if it holds a NaN or is greater in the (real, imaginary)
// order, else the second (utils/math_utils.hpp:99-131: max_complex / min_complex).
template <class A, class B> struct MaximumOp {
    using R = std::conditional_t<std::is_same_v<A, B>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_cplx_v<A>) return (is_nan(a) || cx::c_less(b, a)) ? a : b;
        else if constexpr (is_bool_v<A>) return bool_t(a.v || b.v);
        else if constexpr (is_fp_v<A>) {
            auto x = up(a), y = up(b);
            return (x != x || x >= y) ? a : b;
        }
        else return a >= b ? a : b;
    }
};

template <class A, class B> struct MinimumOp {
    using R = std::conditional_t<std::is_same_v<A, B>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_cplx_v<A>) return (is_nan(a) || cx::c_less(a, b)) ? a : b;
        else if constexpr (is_bool_v<A>) return bool_t(a.v && b.v);
        else if constexpr (is_fp_v<A>) {
            auto x = up(a), y = up(b);
            return (x != x || x <= y) ? a : b;
        }
        else return a <= b ? a : b;
    }
};

// Comparisons: identical types, plus the mixed (int64, uint64) pairs compared
// without loss of range (less.hpp:60-101).
template <class A, class B>
inline constexpr bool cmp_pair_v =
    std::is_same_v<A, B> || (std::is_same_v<A, int64_t> && std::is_same_v<B, uint64_t>) ||
    (std::is_same_v<A, uint64_t> && std::is_same_v<B, int64_t>);

enum CmpKind { CMP_EQ, CMP_NE, CMP_LT, CMP_LE, CMP_GT, CMP_GE };

template <int K, class X, class Y> DPB_D bool cmp_scalar(X x, Y y)
{
    if constexpr (K == CMP_EQ) return x == y;
    else if constexpr (K == CMP_NE) return x != y;
    else if constexpr (K == CMP_LT) return x < y;
    else if constexpr (K == CMP_LE) return x <= y;
    else if constexpr (K == CMP_GT) return x > y;
    else return x >= y;
}

template <int K, class A, class B> struct CompareOp {
    static constexpr bool ordered = (K != CMP_EQ && K != CMP_NE);
    using R = std::conditional_t<cmp_pair_v<A, B>, bool_t, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_cplx_v<A>) {
            // ordered comparisons of complex numbers: real parts decide unless equal, then the
            // imaginary parts; false whenever a NaN is involved (less.hpp:60-101)
            if constexpr (K == CMP_LT) return bool_t(cx::c_less(a, b));
            else if constexpr (K == CMP_LE) return bool_t(cx::c_less_equal(a, b));
            else if constexpr (K == CMP_GT) return bool_t(cx::c_less(b, a));
            else if constexpr (K == CMP_GE) return bool_t(cx::c_less_equal(b, a));
            else {
                bool eq = (a.re == b.re) && (a.im == b.im);
                return bool_t(K == CMP_EQ ? eq : !eq);
            }
        }
        else if constexpr (is_bool_v<A>) {
            return bool_t(cmp_scalar<K>(int(a.v != 0), int(b.v != 0)));
        }
        else if constexpr (std::is_same_v<A, int64_t> && std::is_same_v<B, uint64_t>) {
            // a negative left operand is smaller than every unsigned value
            if (a < 0) return bool_t(K == CMP_NE || K == CMP_LT || K == CMP_LE);
            return bool_t(cmp_scalar<K>(static_cast<uint64_t>(a), b));
        }
        else if constexpr (std::is_same_v<A, uint64_t> && std::is_same_v<B, int64_t>) {
            if (b < 0) return bool_t(K == CMP_NE || K == CMP_GT || K == CMP_GE);
            return bool_t(cmp_scalar<K>(a, static_cast<uint64_t>(b)));
        }
        else {
            return bool_t(cmp_scalar<K>(up(a), up(b)));
        }
    }
};
template <class A, class B> using EqualOp = CompareOp<CMP_EQ, A, B>;
template <class A, class B> using NotEqualOp = CompareOp<CMP_NE, A, B>;
template <class A, class B> using LessOp = CompareOp<CMP_LT, A, B>;
template <class A, class B> using LessEqualOp = CompareOp<CMP_LE, A, B>;
template <class A, class B> using GreaterOp = CompareOp<CMP_GT, A, B>;
template <class A, class B> using GreaterEqualOp = CompareOp<CMP_GE, A, B>;

template <class A, class B> struct LogicalAndOp {
    using R = std::conditional_t<std::is_same_v<A, B>, bool_t, NoType>;
    static DPB_D R apply(A a, B b)
    {
        return bool_t(static_cast<bool>(convert<bool_t>(a)) && static_cast<bool>(convert<bool_t>(b)));
    }
};

template <class A, class B> struct LogicalOrOp {
    using R = std::conditional_t<std::is_same_v<A, B>, bool_t, NoType>;
    static DPB_D R apply(A a, B b)
    {
        return bool_t(static_cast<bool>(convert<bool_t>(a)) || static_cast<bool>(convert<bool_t>(b)));
    }
};

// pow (pow.hpp:63-114): integers by repeated squaring with wrap-around, a negative exponent gives
// 0; floating types through the library pow; complex through integer powers / exp(b log a)
template <class A, class B> struct PowOp {
    using R = std::conditional_t<std::is_same_v<A, B> && (is_fp_v<A> || is_int_v<A> || is_cplx_v<A>), A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_int_v<A>) {
            if constexpr (std::is_signed_v<B>) { if (b < B(0)) return A(0); }
            using U = std::make_unsigned_t<A>;
            U base = static_cast<U>(a), res = 1;
            if (a == A(1) || b == B(0)) return A(1);
            std::make_unsigned_t<B> e = static_cast<std::make_unsigned_t<B>>(b);
            while (e > 0) {
                if (e & 1) res = static_cast<U>(res * base);
                e >>= 1;
                base = static_cast<U>(base * base);
            }
            return static_cast<A>(res);
        }
        else if constexpr (is_cplx_v<A>) return cx::c_pow(a, b);
        else if constexpr (std::is_same_v<A, double>) return pow(a, b);
        else if constexpr (std::is_same_v<A, float>) return powf(a, b);
        else return __float2half(powf(__half2float(a), __half2float(b)));
    }
};


// ===================================================================== more unary
// Floating-point functions of one argument; float16 is computed in float32.
#define DPB_FP_UNARY2(NAME, EXPR_F, EXPR_D)                                      \
    template <class T> struct NAME {                                             \
        using R = std::conditional_t<is_fp_v<T>, T, NoType>;                     \
        static DPB_D R apply(T v)                                                \
        {                                                                        \
            if constexpr (std::is_same_v<T, double>) { const double x = v; return (EXPR_D); } \
            else if constexpr (std::is_same_v<T, float>) { const float x = v; return (EXPR_F); } \
            else { const float x = __half2float(v); return __float2half(EXPR_F); } \
        }                                                                        \
    };
// the same with a complex branch
#define DPB_FP_UNARY2C(NAME, EXPR_F, EXPR_D, FN_C)                               \
    template <class T> struct NAME {                                             \
        using R = std::conditional_t<is_fp_v<T> || is_cplx_v<T>, T, NoType>;     \
        static DPB_D R apply(T v)                                                \
        {                                                                        \
            if constexpr (is_cplx_v<T>) return cx::FN_C(v);                      \
            else if constexpr (std::is_same_v<T, double>) { const double x = v; return (EXPR_D); } \
            else if constexpr (std::is_same_v<T, float>) { const float x = v; return (EXPR_F); } \
            else { const float x = __half2float(v); return __float2half(EXPR_F); } \
        }                                                                        \
    };

DPB_FP_UNARY2C(AcosOp, acosf(x), acos(x), c_acos)       // acos.hpp
DPB_FP_UNARY2C(AcoshOp, acoshf(x), acosh(x), c_acosh)   // acosh.hpp
DPB_FP_UNARY2C(AsinOp, asinf(x), asin(x), c_asin)       // asin.hpp
DPB_FP_UNARY2C(AsinhOp, asinhf(x), asinh(x), c_asinh)   // asinh.hpp
DPB_FP_UNARY2C(AtanOp, atanf(x), atan(x), c_atan)       // atan.hpp
DPB_FP_UNARY2C(AtanhOp, atanhf(x), atanh(x), c_atanh)   // atanh.hpp
DPB_FP_UNARY2(CbrtOp, cbrtf(x), cbrt(x))                // cbrt.hpp
DPB_FP_UNARY2C(CoshOp, coshf(x), cosh(x), c_cosh)       // cosh.hpp
DPB_FP_UNARY2C(SinhOp, sinhf(x), sinh(x), c_sinh)       // sinh.hpp
DPB_FP_UNARY2C(TanOp, tanf(x), tan(x), c_tan)           // tan.hpp
DPB_FP_UNARY2C(Exp2Op, exp2f(x), exp2(x), c_exp2)       // exp2.hpp
DPB_FP_UNARY2C(Log2Op, log2f(x), log2(x), c_log2)       // log2.hpp
DPB_FP_UNARY2C(Log10Op, log10f(x), log10(x), c_log10)   // log10.hpp
// rsqrt.hpp: reciprocal of the correctly rounded square root
DPB_FP_UNARY2(RsqrtOp, 1.0f / sqrtf(x), 1.0 / sqrt(x))
#undef DPB_FP_UNARY2C
#undef DPB_FP_UNARY2

// trunc.hpp / round.hpp (round half to even): identity on integers
template <class T> struct TruncOp {
    using R = std::conditional_t<is_cplx_v<T> || is_bool_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_half_v<T>) return htrunc(x);
        else if constexpr (std::is_floating_point_v<T>) return trunc(x);
        else return x;
    }
};

template <class T> struct RoundOp {
    using R = std::conditional_t<is_bool_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return T(rint(x.re), rint(x.im));
        else if constexpr (is_half_v<T>) return hrint(x);
        else if constexpr (std::is_floating_point_v<T>) return rint(x);
        else return x;
    }
};

// signbit.hpp: floating types only
template <class T> struct SignbitOp {
    using R = std::conditional_t<is_fp_v<T>, bool_t, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_half_v<T>) return bool_t((__half_as_ushort(x) & 0x8000u) != 0);
        else return bool_t(signbit(x));
    }
};

// bitwise_invert.hpp: logical not for bool, complement for integers
template <class T> struct BitwiseInvertOp {
    using R = std::conditional_t<is_bool_v<T> || is_int_v<T>, T, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_bool_v<T>) return bool_t(!x.v);
        else return static_cast<T>(~x);
    }
};

// conj.hpp (bool -> int8), real.hpp, imag.hpp (real types: the value itself / zero)
template <class T> struct ConjOp {
    using R = std::conditional_t<is_bool_v<T>, int8_t, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_bool_v<T>) return x.v ? int8_t(1) : int8_t(0);
        else if constexpr (is_cplx_v<T>) return T(x.re, -x.im);
        else return x;
    }
};

template <class T> struct RealOp {
    using R = real_of_t<T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return x.re;
        else return x;
    }
};

template <class T> struct ImagOp {
    using R = real_of_t<T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return x.im;
        else if constexpr (is_bool_v<T>) return bool_t(false);
        else if constexpr (is_half_v<T>) return __float2half(0.0f);
        else return T(0);
    }
};

// angle.hpp, proj.hpp: complex types only
template <class T> struct AngleOp {
    using R = std::conditional_t<is_cplx_v<T>, real_of_t<T>, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) return atan2(x.im, x.re);
        else return R{};
    }
};

template <class T> struct ProjOp {
    using R = std::conditional_t<is_cplx_v<T>, T, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_cplx_v<T>) {
            using F = real_of_t<T>;
            if (isinf(x.re) || isinf(x.im)) return T(F(INFINITY), copysign(F(0), x.im));
            return x;
        }
        else return R{};
    }
};

// ==================================================================== more binary
#define DPB_FP_BINARY(NAME, EXPR_F, EXPR_D)                                      \
    template <class A, class B> struct NAME {                                    \
        using R = std::conditional_t<std::is_same_v<A, B> && is_fp_v<A>, A, NoType>; \
        static DPB_D R apply(A a, B b)                                           \
        {                                                                        \
            if constexpr (std::is_same_v<A, double>) { const double x = a, y = b; return (EXPR_D); } \
            else if constexpr (std::is_same_v<A, float>) { const float x = a, y = b; return (EXPR_F); } \
            else { const float x = __half2float(a), y = __half2float(b); return __float2half(EXPR_F); } \
        }                                                                        \
    };

template <class F> DPB_D F logaddexp_impl(F x, F y)
{
    // utils/math_utils.hpp:131-147
    if (x == y) return x + log(F(2));
    const F d = x - y;
    return d > F(0) ? x + log1p(exp(-d)) : (d <= F(0) ? y + log1p(exp(d)) : F(NAN));
}

DPB_FP_BINARY(Atan2Op, atan2f(x, y), atan2(x, y))               // atan2.hpp
DPB_FP_BINARY(HypotOp, hypotf(x, y), hypot(x, y))               // hypot.hpp
DPB_FP_BINARY(CopysignOp, copysignf(x, y), copysign(x, y))      // copysign.hpp
DPB_FP_BINARY(LogaddexpOp, logaddexp_impl<float>(x, y), logaddexp_impl<double>(x, y))  // logaddexp.hpp
#undef DPB_FP_BINARY

// nextafter.hpp: float16 steps in its own format
template <class A, class B> struct NextafterOp {
    using R = std::conditional_t<std::is_same_v<A, B> && is_fp_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (std::is_same_v<A, double>) return (a == b) ? b : nextafter(a, b);
        else if constexpr (std::is_same_v<A, float>) return (a == b) ? b : nextafterf(a, b);
        else {
            const float x = __half2float(a), y = __half2float(b);
            if (x != x || y != y) return __float2half(x + y);
            if (x == y) return b;
            unsigned short u = __half_as_ushort(a);
            if (x == 0.0f) return __ushort_as_half(static_cast<unsigned short>((y < 0.0f ? 0x8000u : 0u) | 1u));
            const bool away = (y > x) == (x > 0.0f);   // magnitude grows
            u = static_cast<unsigned short>(away ? u + 1 : u - 1);
            return __ushort_as_half(u);
        }
    }
};

// bitwise_and.hpp / bitwise_or.hpp / bitwise_xor.hpp: bool and integers, identical types
enum BitKind { BIT_AND, BIT_OR, BIT_XOR };
template <int K, class A, class B> struct BitwiseOp {
    using R = std::conditional_t<std::is_same_v<A, B> && (is_bool_v<A> || is_int_v<A>), A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_bool_v<A>) {
            if constexpr (K == BIT_AND) return bool_t(a.v && b.v);
            else if constexpr (K == BIT_OR) return bool_t(a.v || b.v);
            else return bool_t(bool(a.v) != bool(b.v));
        }
        else {
            if constexpr (K == BIT_AND) return static_cast<A>(a & b);
            else if constexpr (K == BIT_OR) return static_cast<A>(a | b);
            else return static_cast<A>(a ^ b);
        }
    }
};
template <class A, class B> using BitwiseAndOp = BitwiseOp<BIT_AND, A, B>;
template <class A, class B> using BitwiseOrOp = BitwiseOp<BIT_OR, A, B>;
template <class A, class B> using BitwiseXorOp = BitwiseOp<BIT_XOR, A, B>;

// bitwise_left_shift.hpp:88-104 / bitwise_right_shift.hpp:87-105: a negative count or one of at
// least the bit width gives 0 (right shift of a negative value: -1)
template <class A, class B> struct LeftShiftOp {
    using R = std::conditional_t<std::is_same_v<A, B> && is_int_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        constexpr int bits = static_cast<int>(sizeof(A) * 8);
        if constexpr (std::is_signed_v<B>) { if (b < B(0)) return A(0); }
        if (static_cast<uint64_t>(b) >= static_cast<uint64_t>(bits)) return A(0);
        using U = std::make_unsigned_t<A>;
        return static_cast<A>(static_cast<U>(static_cast<U>(a) << static_cast<int>(b)));
    }
};

template <class A, class B> struct RightShiftOp {
    using R = std::conditional_t<std::is_same_v<A, B> && is_int_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        constexpr int bits = static_cast<int>(sizeof(A) * 8);
        if constexpr (std::is_signed_v<B>) { if (b < B(0)) return A(0); }
        if (static_cast<uint64_t>(b) >= static_cast<uint64_t>(bits)) {
            if constexpr (std::is_signed_v<A>) return a < A(0) ? A(-1) : A(0);
            else return A(0);
        }
        return static_cast<A>(a >> static_cast<int>(b));
    }
};

// floor_divide.hpp / remainder.hpp: integers (division by zero gives 0) and floating types,
// results follow the sign of the divisor
template <class A, class B> struct FloorDivideOp {
    using R = std::conditional_t<std::is_same_v<A, B> && (is_int_v<A> || is_fp_v<A>), A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_int_v<A>) {
            if (b == B(0)) return A(0);
            if constexpr (std::is_signed_v<A>) {
                if (b == B(-1)) return static_cast<A>(A(0) - static_cast<std::make_unsigned_t<A>>(a));
                const A q = static_cast<A>(a / b), m = static_cast<A>(a % b);
                return static_cast<A>(q - ((m != 0 && ((m < 0) != (b < 0))) ? 1 : 0));
            }
            else return static_cast<A>(a / b);
        }
        else {
            const auto x = up(a), y = up(b);
            const auto q = x / y;
            using C = decltype(q);
            return down<A>(q == C(0) ? q : floor(q));
        }
    }
};

template <class A, class B> struct RemainderOp {
    using R = std::conditional_t<std::is_same_v<A, B> && (is_int_v<A> || is_fp_v<A>), A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_int_v<A>) {
            if (b == B(0)) return A(0);
            if constexpr (std::is_signed_v<A>) {
                if (b == B(-1)) return A(0);
                A m = static_cast<A>(a % b);
                if (m != 0 && ((a < 0) != (b < 0))) m = static_cast<A>(m + b);
                return m;
            }
            else return static_cast<A>(a % b);
        }
        else {
            const auto x = up(a), y = up(b);
            auto r = fmod(x, y);
            using C = decltype(r);
            if (r != C(0)) {
                if ((y < C(0)) != (r < C(0))) r += y;
            }
            else r = copysign(C(0), y);
            return down<A>(r);
        }
    }
};

template <class A, class B> struct LogicalXorOp {
    using R = std::conditional_t<std::is_same_v<A, B>, bool_t, NoType>;
    static DPB_D R apply(A a, B b)
    {
        return bool_t(static_cast<bool>(convert<bool_t>(a)) != static_cast<bool>(convert<bool_t>(b)));
    }
};

}  // namespace dpb
