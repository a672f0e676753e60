// Max and min reductions (same input and output type; complex values in the (real, imaginary) order).
#include "reduce_register.cuh"
namespace dpb {
template <int TN> static void reg_minmax_one(RedTables &t)
{
    using T = type_of_t<TN>;
    {
        t.reduce[DPB_R_MAX][TN][TN] = &red_entry<ExtremeRed<true, T, T>>;
        t.reduce[DPB_R_MIN][TN][TN] = &red_entry<ExtremeRed<false, T, T>>;
    }
}
template <int... TN> static void reg_minmax(RedTables &t, std::integer_sequence<int, TN...>)
{
    (reg_minmax_one<TN>(t), ...);
}
void register_reduce_minmax(RedTables &t)
{
    reg_minmax(t, std::make_integer_sequence<int, DPB_NUM_TYPES>());
}
}  // namespace dpb
