// maximum, minimum, logical_and, logical_or, pow.
#include "ew_register.cuh"
namespace dpb {
void register_binary_misc(EwTables &t)
{
    reg_binary<MaximumOp>(t, DPB_B_MAXIMUM);
    reg_binary<MinimumOp>(t, DPB_B_MINIMUM);
    reg_binary<LogicalAndOp>(t, DPB_B_LOGICAL_AND);
    reg_binary<LogicalOrOp>(t, DPB_B_LOGICAL_OR);
    reg_binary<PowOp>(t, DPB_B_POW);
}
}  // namespace dpb
