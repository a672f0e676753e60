// Dispatch tables of the elementwise engine and the helpers that fill them.
// One table entry = one instantiation of launch_ew for a functor; entries are
// looked up by (operation, argument type ids), the way the reference indexes
// its [14][14] function-pointer tables built by DispatchTableBuilder
// (dpnp/tensor/libtensor/include/utils/type_dispatch_building.hpp:64-123).
#pragma once

#include <utility>

#include "ew_kernels.cuh"
#include "ew_ops.cuh"

namespace dpb {

typedef int (*ew_fn_t)(const EwPlan &plan, const void *const *in, void *out, cudaStream_t stream);

struct EwEntry {
    ew_fn_t fn = nullptr;
    int rtype = -1;
};

struct EwTables {
    EwEntry unary[DPB_U_NUM_OPS][DPB_NUM_TYPES];
    EwEntry binary[DPB_B_NUM_OPS][DPB_NUM_TYPES][DPB_NUM_TYPES];
    // where: [condition type][log2 of value size in bytes (0..4)]
    ew_fn_t where_[DPB_NUM_TYPES][5];
    // copy/cast: [source type][destination type]
    ew_fn_t cast[DPB_NUM_TYPES][DPB_NUM_TYPES];
};

const EwTables &ew_tables();

// registration functions, one per translation unit
void register_unary_arith(EwTables &t);
void register_unary_math(EwTables &t);
void register_unary_pred(EwTables &t);
void register_binary_arith(EwTables &t);
void register_binary_misc(EwTables &t);
void register_binary_cmp_a(EwTables &t);
void register_binary_cmp_b(EwTables &t);
void register_unary_math2(EwTables &t);
void register_unary_misc2(EwTables &t);
void register_binary_fp2(EwTables &t);
void register_binary_bits(EwTables &t);
void register_binary_divmod(EwTables &t);
void register_where(EwTables &t);
void register_cast_a(EwTables &t);
void register_cast_b(EwTables &t);

template <class F>
int ew_entry(const EwPlan &plan, const void *const *in, void *out, cudaStream_t stream)
{
    return launch_ew(F(), plan, in, out, stream);
}

// 16-byte accesses per thread of the contiguous kernel: an operator may ask for fewer (kUnroll)
template <class O, class = void> struct op_unroll { static constexpr int value = 8; };
template <class O> struct op_unroll<O, std::void_t<decltype(O::kUnroll)>> { static constexpr int value = O::kUnroll; };

template <template <class> class Op, class T> struct UnaryF {
    static constexpr int NIN = 1;
    static constexpr int kUnroll = op_unroll<Op<T>>::value;
    using In0 = T;
    using In1 = char;
    using In2 = char;
    using Out = typename Op<T>::R;
    DPB_D Out operator()(In0 x) const { return Op<T>::apply(x); }
};

template <template <class, class> class Op, class A, class B> struct BinaryF {
    static constexpr int NIN = 2;
    using In0 = A;
    using In1 = B;
    using In2 = char;
    using Out = typename Op<A, B>::R;
    DPB_D Out operator()(In0 x, In1 y) const { return Op<A, B>::apply(x, y); }
};

// opaque value of a given size, used where the operation only moves bits; the payload is
// a machine word (or two) so that copies compile to register moves
template <int BYTES> struct blob_word { using type = unsigned char; static constexpr int N = BYTES; };
template <> struct blob_word<2> { using type = uint16_t; static constexpr int N = 1; };
template <> struct blob_word<4> { using type = uint32_t; static constexpr int N = 1; };
template <> struct blob_word<8> { using type = uint64_t; static constexpr int N = 1; };
template <> struct blob_word<16> { using type = uint64_t; static constexpr int N = 2; };
template <int BYTES> struct alignas(BYTES) blob_t {
    typename blob_word<BYTES>::type w[blob_word<BYTES>::N];
};

template <class C, int BYTES> struct WhereF {
    static constexpr int NIN = 3;
    using In0 = C;
    using In1 = blob_t<BYTES>;
    using In2 = blob_t<BYTES>;
    using Out = blob_t<BYTES>;
    DPB_D Out operator()(In0 c, const In1 &x, const In2 &y) const
    {
        return static_cast<bool>(convert<bool_t>(c)) ? x : y;
    }
};

template <class S, class D> struct CastF {
    static constexpr int NIN = 1;
    using In0 = S;
    using In1 = char;
    using In2 = char;
    using Out = D;
    DPB_D Out operator()(In0 x) const { return convert<D>(x); }
};

template <int BYTES> struct CopyF {
    static constexpr int NIN = 1;
    using In0 = blob_t<BYTES>;
    using In1 = char;
    using In2 = char;
    using Out = blob_t<BYTES>;
    DPB_D Out operator()(const In0 &x) const { return x; }
};

template <class T> struct DivScalarF {
    static constexpr int NIN = 1;
    using In0 = T;
    using In1 = char;
    using In2 = char;
    using Out = T;
    compute_t<T> s;
    DPB_D Out operator()(In0 x) const { return down<T>(up(x) / s); }
};

template <int BYTES> struct FillF {
    static constexpr int NIN = 0;
    using In0 = char;
    using In1 = char;
    using In2 = char;
    using Out = blob_t<BYTES>;
    Out v;
    DPB_D Out operator()() const { return v; }
};

// ------------------------------------------------------- table population
template <template <class> class Op, int TN> void reg_unary_one(EwEntry *row)
{
    using T = type_of_t<TN>;
    using R = typename Op<T>::R;
    if constexpr (!std::is_same_v<R, NoType>) {
        row[TN].fn = &ew_entry<UnaryF<Op, T>>;
        row[TN].rtype = typenum_of<R>::value;
    }
}
template <template <class> class Op, int... TN>
void reg_unary_seq(EwEntry *row, std::integer_sequence<int, TN...>)
{
    (reg_unary_one<Op, TN>(row), ...);
}
template <template <class> class Op> void reg_unary(EwTables &t, int op)
{
    reg_unary_seq<Op>(t.unary[op], std::make_integer_sequence<int, DPB_NUM_TYPES>());
}

template <template <class, class> class Op, int TA, int TB>
void reg_binary_one(EwEntry (*tab)[DPB_NUM_TYPES])
{
    using A = type_of_t<TA>;
    using B = type_of_t<TB>;
    using R = typename Op<A, B>::R;
    if constexpr (!std::is_same_v<R, NoType>) {
        tab[TA][TB].fn = &ew_entry<BinaryF<Op, A, B>>;
        tab[TA][TB].rtype = typenum_of<R>::value;
    }
}
template <template <class, class> class Op, int TA, int... TB>
void reg_binary_row(EwEntry (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TB...>)
{
    (reg_binary_one<Op, TA, TB>(tab), ...);
}
template <template <class, class> class Op, int... TA>
void reg_binary_seq(EwEntry (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TA...>)
{
    (reg_binary_row<Op, TA>(tab, std::make_integer_sequence<int, DPB_NUM_TYPES>()), ...);
}
template <template <class, class> class Op> void reg_binary(EwTables &t, int op)
{
    reg_binary_seq<Op>(t.binary[op], std::make_integer_sequence<int, DPB_NUM_TYPES>());
}

}  // namespace dpb
