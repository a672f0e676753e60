// Elementwise operation functors.  Each functor template takes the argument
// element type(s) and exposes
//   R      - result element type, or NoType when the combination has no kernel
//   apply  - the scalar operation
// The supported type maps follow the *OutputType tables of the reference
// (dpnp/tensor/libtensor/include/kernels/elementwise_functions/<op>.hpp).
#pragma once

#include <math.h>

#include "common.cuh"

namespace dpb {

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

#define DPB_FP_UNARY(NAME, FN_F, FN_D)                                           \
    template <class T> struct NAME {                                             \
        using R = std::conditional_t<is_fp_v<T>, T, NoType>;                     \
        static DPB_D R apply(T x)                                                \
        {                                                                        \
            if constexpr (std::is_same_v<T, double>) return FN_D(x);             \
            else if constexpr (std::is_same_v<T, float>) return FN_F(x);         \
            else return __float2half(FN_F(__half2float(x)));                     \
        }                                                                        \
    };

DPB_FP_UNARY(ExpOp, expf, exp)
DPB_FP_UNARY(LogOp, logf, log)
DPB_FP_UNARY(SqrtOp, sqrtf, sqrt)
DPB_FP_UNARY(SinOp, sinf, sin)
DPB_FP_UNARY(CosOp, cosf, cos)
DPB_FP_UNARY(TanhOp, tanhf, tanh)
DPB_FP_UNARY(Expm1Op, expm1f, expm1)
DPB_FP_UNARY(Log1pOp, log1pf, log1p)
#undef DPB_FP_UNARY

template <class T> struct ReciprocalOp {
    using R = std::conditional_t<is_fp_v<T>, T, NoType>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_half_v<T>) return __float2half(1.0f / __half2float(x));
        else return T(1) / x;
    }
};

// erf: float16 input is promoted to float32
// (dpnp/backend/extensions/ufunc/elementwise_functions/erf_funcs.cpp:73-85)
template <class T> struct ErfOp {
    using R = std::conditional_t<is_half_v<T>, float, std::conditional_t<is_fp_v<T>, T, NoType>>;
    static DPB_D R apply(T x)
    {
        if constexpr (std::is_same_v<T, double>) return erf(x);
        else if constexpr (std::is_same_v<T, float>) return erff(x);
        else return erff(__half2float(x));
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
    using R = std::conditional_t<is_bool_v<T> || is_cplx_v<T>, NoType, T>;
    static DPB_D R apply(T x)
    {
        if constexpr (is_uint_v<T>) return static_cast<T>(x > 0 ? 1 : 0);
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

// true_divide: floating types only (integers are promoted to the default
// floating type by the caller, dpnp/tensor/_type_utils.py:89-107).
template <class A, class B> struct TrueDivideOp {
    using R = std::conditional_t<std::is_same_v<A, B> && is_fp_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_half_v<A>) return __float2half(__half2float(a) / __half2float(b));
        else return a / b;
    }
};

// maximum / minimum propagate NaN (first NaN operand wins).
template <class A, class B> struct MaximumOp {
    using R = std::conditional_t<std::is_same_v<A, B> && !is_cplx_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_bool_v<A>) return bool_t(a.v || b.v);
        else if constexpr (is_fp_v<A>) {
            auto x = up(a), y = up(b);
            return (x != x || x >= y) ? a : b;
        }
        else return a >= b ? a : b;
    }
};

template <class A, class B> struct MinimumOp {
    using R = std::conditional_t<std::is_same_v<A, B> && !is_cplx_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_bool_v<A>) return bool_t(a.v && b.v);
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
    using R = std::conditional_t<cmp_pair_v<A, B> && !(ordered && is_cplx_v<A>), bool_t, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (is_cplx_v<A>) {
            bool eq = (a.re == b.re) && (a.im == b.im);
            return bool_t(K == CMP_EQ ? eq : !eq);
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

// pow: floating types only in this build
template <class A, class B> struct PowOp {
    using R = std::conditional_t<std::is_same_v<A, B> && is_fp_v<A>, A, NoType>;
    static DPB_D R apply(A a, B b)
    {
        if constexpr (std::is_same_v<A, double>) return pow(a, b);
        else if constexpr (std::is_same_v<A, float>) return powf(a, b);
        else return __float2half(powf(__half2float(a), __half2float(b)));
    }
};

}  // namespace dpb
