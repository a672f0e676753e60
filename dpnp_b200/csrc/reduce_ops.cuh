// Reduction operators.  A reduction operator R describes
//   R::In      element type read from memory
//   R::Acc     accumulator type carried through the tree (also the type of
//              the partial results between the two passes)
//   R::Out     element type written to the result
//   identity() neutral accumulator
//   load(v, i) accumulator for element v found at reduction index i
//   combine    associative, commutative merge of two accumulators
//   finish     accumulator -> result element
//   R::Stage2  the operator that merges partial accumulators (In = Acc)
//
// Semantics follow the reference: sums of bool into bool are logical-or
// (source/reductions/sum.cpp:268-270), floating max/min propagate NaN
// (include/utils/sycl_utils.hpp:332-376), argmax/argmin return the smallest
// index among equal extremes and treat NaN as the extreme
// (include/kernels/reductions.hpp:1917-1971,2062-2117; source/reductions/argmax.cpp:139-141),
// identities as in sycl_utils.hpp:380-571.
#pragma once

#include <limits>

#include "common.cuh"
#include "ew_ops.cuh"

namespace dpb {

// accumulate half in float
template <class Out> struct acc_of { using type = Out; };
template <> struct acc_of<half_t> { using type = float; };
template <class Out> using acc_of_t = typename acc_of<Out>::type;

template <class T> DPB_HD T lowest_value()
{
    if constexpr (is_cplx_v<T>) return T(lowest_value<real_of_t<T>>(), lowest_value<real_of_t<T>>());
    else if constexpr (std::is_same_v<T, float>) return -INFINITY;
    else if constexpr (std::is_same_v<T, double>) return -static_cast<double>(INFINITY);
    else if constexpr (is_bool_v<T>) return bool_t(false);
    else return std::numeric_limits<T>::lowest();
}
template <class T> DPB_HD T highest_value()
{
    if constexpr (is_cplx_v<T>) return T(highest_value<real_of_t<T>>(), highest_value<real_of_t<T>>());
    else if constexpr (std::is_same_v<T, float>) return INFINITY;
    else if constexpr (std::is_same_v<T, double>) return static_cast<double>(INFINITY);
    else if constexpr (is_bool_v<T>) return bool_t(true);
    else return std::numeric_limits<T>::max();
}

// ----------------------------------------------------------- sum and prod
template <class TIn, class TOut, class TAcc = acc_of_t<TOut>> struct SumRed {
    using In = TIn;
    using Acc = TAcc;
    using Out = TOut;
    using Stage2 = SumRed<Acc, TOut, Acc>;
    static constexpr bool kVectorStep = false;
    static DPB_D Acc identity()
    {
        if constexpr (is_cplx_v<Acc>) return Acc(0, 0);
        else if constexpr (is_bool_v<Acc>) return bool_t(false);
        else return Acc(0);
    }
    static DPB_D Acc load(In v, int64_t) { return convert<Acc>(v); }
    static DPB_D Acc step(Acc a, In v, int64_t i) { return combine(a, load(v, i)); }
    static DPB_D Acc combine(Acc a, Acc b)
    {
        if constexpr (is_bool_v<Acc>) return bool_t(a.v || b.v);
        else if constexpr (is_cplx_v<Acc>) return Acc(a.re + b.re, a.im + b.im);
        else return static_cast<Acc>(a + b);
    }
    static DPB_D Out finish(Acc a) { return convert<Out>(a); }
};

template <class TIn, class TOut, class TAcc = acc_of_t<TOut>> struct ProdRed {
    using In = TIn;
    using Acc = TAcc;
    using Out = TOut;
    using Stage2 = ProdRed<Acc, TOut, Acc>;
    static constexpr bool kVectorStep = false;
    static DPB_D Acc identity()
    {
        if constexpr (is_cplx_v<Acc>) return Acc(1, 0);
        else if constexpr (is_bool_v<Acc>) return bool_t(true);
        else return Acc(1);
    }
    static DPB_D Acc load(In v, int64_t) { return convert<Acc>(v); }
    static DPB_D Acc step(Acc a, In v, int64_t i) { return combine(a, load(v, i)); }
    static DPB_D Acc combine(Acc a, Acc b)
    {
        if constexpr (is_bool_v<Acc>) return bool_t(a.v && b.v);
        else if constexpr (is_cplx_v<Acc>)
            return Acc(a.re * b.re - a.im * b.im, a.re * b.im + a.im * b.re);
        else return static_cast<Acc>(a * b);
    }
    static DPB_D Out finish(Acc a) { return convert<Out>(a); }
};

// ------------------------------------------------- logsumexp and hypot
// Floating types only (source/reductions/logsumexp.cpp, reduce_hypot.cpp); the merge of two
// accumulators is the elementwise logaddexp / hypot (include/utils/sycl_utils.hpp:574-640).
template <class TIn, class TOut, class TAcc = acc_of_t<TOut>> struct LogSumExpRed {
    using In = TIn;
    using Acc = TAcc;
    using Out = TOut;
    using Stage2 = LogSumExpRed<Acc, TOut, Acc>;
    static constexpr bool kVectorStep = false;
    static DPB_D Acc identity() { return -static_cast<Acc>(INFINITY); }
    static DPB_D Acc load(In v, int64_t) { return convert<Acc>(v); }
    static DPB_D Acc step(Acc a, In v, int64_t i) { return combine(a, load(v, i)); }
    static DPB_D Acc combine(Acc a, Acc b) { return logaddexp_impl<Acc>(a, b); }
    static DPB_D Out finish(Acc a) { return convert<Out>(a); }
};

template <class TIn, class TOut, class TAcc = acc_of_t<TOut>> struct HypotRed {
    using In = TIn;
    using Acc = TAcc;
    using Out = TOut;
    using Stage2 = HypotRed<Acc, TOut, Acc>;
    static constexpr bool kVectorStep = false;
    static DPB_D Acc identity() { return Acc(0); }
    static DPB_D Acc load(In v, int64_t) { return convert<Acc>(v); }
    static DPB_D Acc step(Acc a, In v, int64_t i) { return combine(a, load(v, i)); }
    static DPB_D Acc combine(Acc a, Acc b) { return hypot(a, b); }
    static DPB_D Out finish(Acc a) { return convert<Out>(a); }
};

// ------------------------------------------------------------ max and min
// Order helpers shared by max/min and the searches.  Complex values compare by real part, then by
// imaginary part, and a NaN in either part makes the value the extreme
// (include/utils/math_utils.hpp:43-131, include/kernels/reductions.hpp:1914-1963).
template <class V> DPB_D bool sv_nan(const V &v)
{
    if constexpr (is_cplx_v<V>) return v.re != v.re || v.im != v.im;
    else if constexpr (std::is_floating_point_v<V>) return v != v;
    else return false;
}
template <class V> DPB_D bool sv_eq(const V &a, const V &b)
{
    if constexpr (is_cplx_v<V>) return a.re == b.re && a.im == b.im;
    else return a == b;
}
template <bool IS_MAX, class V> DPB_D bool sv_better(const V &a, const V &b)   // NaN-free operands
{
    if constexpr (is_cplx_v<V>) {
        if (a.re == b.re) return IS_MAX ? (a.im > b.im) : (a.im < b.im);
        return IS_MAX ? (a.re > b.re) : (a.re < b.re);
    }
    else return IS_MAX ? (a > b) : (a < b);
}

template <bool IS_MAX, class TIn, class TOut, class TAcc = acc_of_t<TOut>> struct ExtremeRed {
    using In = TIn;
    using Acc = TAcc;
    using Out = TOut;
    using Stage2 = ExtremeRed<IS_MAX, Acc, TOut, Acc>;
    static constexpr bool kVectorStep = false;
    static DPB_D Acc identity() { return IS_MAX ? lowest_value<Acc>() : highest_value<Acc>(); }
    static DPB_D Acc load(In v, int64_t) { return convert<Acc>(v); }
    static DPB_D Acc step(Acc a, In v, int64_t i) { return combine(a, load(v, i)); }
    static DPB_D Acc combine(Acc a, Acc b)
    {
        if constexpr (is_bool_v<Acc>) return IS_MAX ? bool_t(a.v || b.v) : bool_t(a.v && b.v);
        else if constexpr (std::is_floating_point_v<Acc> || is_cplx_v<Acc>) {
            // selects, not early returns: the branches cost more than the compares they skip
            // (the first NaN wins; without NaNs the later operand wins a tie, as before)
            Acc r = sv_better<IS_MAX>(a, b) ? a : b;
            r = sv_nan(b) ? b : r;
            r = sv_nan(a) ? a : r;
            return r;
        }
        else return IS_MAX ? (a > b ? a : b) : (a < b ? a : b);
    }
    static DPB_D Out finish(Acc a) { return convert<Out>(a); }
};

// ------------------------------------------------------ argmax and argmin
template <class V> struct alignas(16) ValIdx {
    V val;
    int64_t idx;
};

// Total order used by the search: NaN beats every number; among equals (and
// among NaNs) the smaller index wins.
template <bool IS_MAX, class V> DPB_D bool search_better(const ValIdx<V> &a, const ValIdx<V> &b)
{
    if constexpr (std::is_floating_point_v<V> || is_cplx_v<V>) {
        const bool an = sv_nan(a.val), bn = sv_nan(b.val);
        if (an || bn) {
            if (an && bn) return a.idx < b.idx;
            return an;
        }
    }
    if (sv_eq(a.val, b.val)) return a.idx < b.idx;
    return sv_better<IS_MAX>(a.val, b.val);
}

template <class V> struct search_val { using type = V; };
template <> struct search_val<half_t> { using type = float; };
template <> struct search_val<bool_t> { using type = uint8_t; };

template <bool IS_MAX, class TIn, class V = typename search_val<TIn>::type, bool STAGE2 = false>
struct SearchRed {
    using In = std::conditional_t<STAGE2, ValIdx<V>, TIn>;
    using Acc = ValIdx<V>;
    using Out = int64_t;
    using Stage2 = SearchRed<IS_MAX, TIn, V, true>;
    // one accumulator per group of adjacent elements: see step_vec
    static constexpr bool kVectorStep = !STAGE2;
    // The identity carries the largest index so that any real element wins a tie.
    static DPB_D Acc identity()
    {
        Acc a;
        a.val = IS_MAX ? lowest_value<V>() : highest_value<V>();
        a.idx = std::numeric_limits<int64_t>::max();
        return a;
    }
    static DPB_D Acc load(const In &v, int64_t i)
    {
        if constexpr (STAGE2) {
            return v;
        }
        else {
            Acc a;
            if constexpr (is_bool_v<TIn>) a.val = v.v ? 1 : 0;
            else a.val = convert<V>(v);
            a.idx = i;
            return a;
        }
    }
    // The pieces of `step` for kernels that keep the value and a short row number in registers and
    // build the accumulator at the end: the value of an element, and whether it replaces the best
    // one seen so far (strictly better; the first NaN beats every number and every later NaN).
    using Val = V;
    static DPB_D V value(const In &v)
    {
        if constexpr (STAGE2) return v.val;
        else if constexpr (is_bool_v<TIn>) return v.v ? 1 : 0;
        else return convert<V>(v);
    }
    static DPB_D bool beats(const V &x, const V &best)
    {
        if constexpr (std::is_floating_point_v<V> || is_cplx_v<V>) {
            const bool bn = sv_nan(best), xn = sv_nan(x), better = sv_better<IS_MAX>(x, best);
            return !bn & (xn | better);       // no short circuit: every test is a compare, not a branch
        }
        else return sv_better<IS_MAX>(x, best);
    }
    // Accumulate one element whose index is larger than every index this
    // accumulator has seen: it wins only if strictly better (or if nothing
    // has been seen yet).
    static DPB_D Acc step(const Acc &a, const In &v, int64_t i)
    {
        if constexpr (STAGE2) {
            return combine(a, v);
        }
        else {
            V x;
            if constexpr (is_bool_v<TIn>) x = v.v ? 1 : 0;
            else x = convert<V>(v);
            bool wins;
            if constexpr (std::is_floating_point_v<V> || is_cplx_v<V>) {
                const bool xn = sv_nan(x), an = sv_nan(a.val);
                wins = an ? false : (xn || sv_better<IS_MAX>(x, a.val));
            }
            else wins = sv_better<IS_MAX>(x, a.val);
            wins = wins || (a.idx == std::numeric_limits<int64_t>::max());
            Acc r = a;
            if (wins) {
                r.val = x;
                r.idx = i;
            }
            return r;
        }
    }
    // Accumulate N adjacent elements starting at index i0.  Only when the best of the
    // group can beat the accumulator (rare once the scan has warmed up, and never for
    // a mere tie) are the elements examined one by one.
    template <int N> static DPB_D Acc step_vec(const Acc &a, const In (&v)[N], int64_t i0)
    {
        if constexpr (is_cplx_v<V>) {
            Acc r = a;
#pragma unroll
            for (int k = 0; k < N; ++k) r = step(r, v[k], i0 + k);
            return r;
        }
        else {
            V x[N];
            bool any_nan = false;
#pragma unroll
            for (int k = 0; k < N; ++k) {
                if constexpr (is_bool_v<TIn>) x[k] = v[k].v ? 1 : 0;
                else x[k] = convert<V>(v[k]);
                if constexpr (std::is_floating_point_v<V>) any_nan = any_nan || (x[k] != x[k]);
            }
            V m = x[0];
#pragma unroll
            for (int k = 1; k < N; ++k) m = IS_MAX ? (x[k] > m ? x[k] : m) : (x[k] < m ? x[k] : m);
            const bool maybe = (IS_MAX ? (m > a.val) : (m < a.val)) || any_nan ||
                               (a.idx == std::numeric_limits<int64_t>::max());
            Acc r = a;
            if (maybe) {
#pragma unroll
                for (int k = 0; k < N; ++k) r = step(r, v[k], i0 + k);
            }
            return r;
        }
    }
    static DPB_D Acc combine(const Acc &a, const Acc &b) { return search_better<IS_MAX>(a, b) ? a : b; }
    static DPB_D Out finish(const Acc &a) { return a.idx; }
};

}  // namespace dpb
