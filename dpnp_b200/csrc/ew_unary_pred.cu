// Unary predicates (boolean result).
#include "ew_register.cuh"
namespace dpb {
void register_unary_pred(EwTables &t)
{
    reg_unary<LogicalNotOp>(t, DPB_U_LOGICAL_NOT);
    reg_unary<IsNanOp>(t, DPB_U_ISNAN);
    reg_unary<IsFiniteOp>(t, DPB_U_ISFINITE);
    reg_unary<IsInfOp>(t, DPB_U_ISINF);
}
}  // namespace dpb
