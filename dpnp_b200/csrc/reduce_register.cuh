// Dispatch tables of the reduction engine.
#pragma once

#include <utility>

#include "reduce_launch.cuh"

namespace dpb {

typedef int (*red_fn_t)(const RedPlan &plan, const void *arg, void *res, cudaStream_t stream);

struct RedTables {
    red_fn_t reduce[DPB_R_NUM_OPS][DPB_NUM_TYPES][DPB_NUM_TYPES];  // [op][in][out]
    red_fn_t search[DPB_S_NUM_OPS][DPB_NUM_TYPES];                 // [op][in]
};

const RedTables &red_tables();
void register_reduce_sum(RedTables &t);
void register_reduce_prod(RedTables &t);
void register_reduce_minmax(RedTables &t);
void register_reduce_search(RedTables &t);
void register_reduce_fp(RedTables &t);

template <class R> int red_entry(const RedPlan &plan, const void *arg, void *res, cudaStream_t stream)
{
    return launch_reduction<R>(plan, arg, res, stream);
}

// (input, output) pairs with a sum/prod kernel: identical types, integers
// and bool into the 64-bit integer of matching signedness, and the next wider
// floating type.  Other pairs are reached through a cast to a temporary by
// the caller, which yields the same values.
template <class I, class O>
inline constexpr bool accumulate_pair_v =
    std::is_same_v<I, O> ||
    (std::is_same_v<O, int64_t> && (is_bool_v<I> || (is_int_v<I> && sizeof(I) < 8))) ||
    (std::is_same_v<O, uint64_t> && (is_bool_v<I> || (is_uint_v<I> && sizeof(I) < 8))) ||
    (std::is_same_v<O, float> && is_half_v<I>) || (std::is_same_v<O, double> && std::is_same_v<I, float>);

template <template <class, class> class Red, int TI, int TO> void reg_accumulate_one(red_fn_t (*tab)[DPB_NUM_TYPES])
{
    using I = type_of_t<TI>;
    using O = type_of_t<TO>;
    if constexpr (accumulate_pair_v<I, O>) tab[TI][TO] = &red_entry<Red<I, O>>;
}
template <template <class, class> class Red, int TI, int... TO>
void reg_accumulate_row(red_fn_t (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TO...>)
{
    (reg_accumulate_one<Red, TI, TO>(tab), ...);
}
template <template <class, class> class Red, int... TI>
void reg_accumulate(red_fn_t (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TI...>)
{
    (reg_accumulate_row<Red, TI>(tab, std::make_integer_sequence<int, DPB_NUM_TYPES>()), ...);
}


// Floating-point-only reductions: identical types, and the next wider floating type.
template <class I, class O>
inline constexpr bool fp_pair_v =
    (is_fp_v<I> && std::is_same_v<I, O>) || (std::is_same_v<O, float> && is_half_v<I>) ||
    (std::is_same_v<O, double> && std::is_same_v<I, float>);
template <template <class, class> class Red, int TI, int TO> void reg_fp_one(red_fn_t (*tab)[DPB_NUM_TYPES])
{
    using I = type_of_t<TI>;
    using O = type_of_t<TO>;
    if constexpr (fp_pair_v<I, O>) tab[TI][TO] = &red_entry<Red<I, O>>;
}
template <template <class, class> class Red> void reg_fp(red_fn_t (*tab)[DPB_NUM_TYPES])
{
    reg_fp_one<Red, DPB_HALF, DPB_HALF>(tab);
    reg_fp_one<Red, DPB_HALF, DPB_FLOAT>(tab);
    reg_fp_one<Red, DPB_FLOAT, DPB_FLOAT>(tab);
    reg_fp_one<Red, DPB_FLOAT, DPB_DOUBLE>(tab);
    reg_fp_one<Red, DPB_DOUBLE, DPB_DOUBLE>(tab);
}

}  // namespace dpb
