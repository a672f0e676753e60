// Product reductions.
#include "reduce_register.cuh"
namespace dpb {
template <class I, class O> using ProdPair = ProdRed<I, O>;
void register_reduce_prod(RedTables &t)
{
    reg_accumulate<ProdPair>(t.reduce[DPB_R_PROD], std::make_integer_sequence<int, DPB_NUM_TYPES>());
}
}  // namespace dpb
