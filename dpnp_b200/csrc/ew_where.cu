// where(condition, x1, x2): the condition may have any type (non-zero is
// true); the values only move, so they are handled by size class.
#include "ew_register.cuh"
namespace dpb {
template <int TC> static void reg_where_one(EwTables &t)
{
    using C = type_of_t<TC>;
    t.where_[TC][0] = &ew_entry<WhereF<C, 1>>;
    t.where_[TC][1] = &ew_entry<WhereF<C, 2>>;
    t.where_[TC][2] = &ew_entry<WhereF<C, 4>>;
    t.where_[TC][3] = &ew_entry<WhereF<C, 8>>;
    t.where_[TC][4] = &ew_entry<WhereF<C, 16>>;
}
template <int... TC> static void reg_where_seq(EwTables &t, std::integer_sequence<int, TC...>)
{
    (reg_where_one<TC>(t), ...);
}
void register_where(EwTables &t)
{
    reg_where_seq(t, std::make_integer_sequence<int, DPB_NUM_TYPES>());
}
}  // namespace dpb
