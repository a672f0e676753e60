// Sum reductions.
#include "reduce_register.cuh"
namespace dpb {
template <class I, class O> using SumPair = SumRed<I, O>;
void register_reduce_sum(RedTables &t)
{
    reg_accumulate<SumPair>(t.reduce[DPB_R_SUM], std::make_integer_sequence<int, DPB_NUM_TYPES>());
}
}  // namespace dpb
