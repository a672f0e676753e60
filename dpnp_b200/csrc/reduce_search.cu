// argmax and argmin.
#include "reduce_register.cuh"
namespace dpb {
template <int TN> static void reg_search_one(RedTables &t)
{
    using T = type_of_t<TN>;
    {
        t.search[DPB_S_ARGMAX][TN] = &red_entry<SearchRed<true, T>>;
        t.search[DPB_S_ARGMIN][TN] = &red_entry<SearchRed<false, T>>;
    }
}
template <int... TN> static void reg_search(RedTables &t, std::integer_sequence<int, TN...>)
{
    (reg_search_one<TN>(t), ...);
}
void register_reduce_search(RedTables &t)
{
    reg_search(t, std::make_integer_sequence<int, DPB_NUM_TYPES>());
}
}  // namespace dpb
