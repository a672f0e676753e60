// less_equal, greater, greater_equal.
#include "ew_register.cuh"
namespace dpb {
void register_binary_cmp_b(EwTables &t)
{
    reg_binary<LessEqualOp>(t, DPB_B_LESS_EQUAL);
    reg_binary<GreaterOp>(t, DPB_B_GREATER);
    reg_binary<GreaterEqualOp>(t, DPB_B_GREATER_EQUAL);
}
}  // namespace dpb
