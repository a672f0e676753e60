// logsumexp and hypot reductions (floating types).
#include "reduce_register.cuh"
namespace dpb {
template <class I, class O> using LogSumExpPair = LogSumExpRed<I, O>;
template <class I, class O> using HypotPair = HypotRed<I, O>;
void register_reduce_fp(RedTables &t)
{
    reg_fp<LogSumExpPair>(t.reduce[DPB_R_LOGSUMEXP]);
    reg_fp<HypotPair>(t.reduce[DPB_R_HYPOT]);
}
}  // namespace dpb
