// Unary arithmetic operations: table entries for every supported type.
#include "ew_register.cuh"
namespace dpb {
void register_unary_arith(EwTables &t)
{
    reg_unary<NegativeOp>(t, DPB_U_NEGATIVE);
    reg_unary<PositiveOp>(t, DPB_U_POSITIVE);
    reg_unary<AbsOp>(t, DPB_U_ABS);
    reg_unary<SquareOp>(t, DPB_U_SQUARE);
    reg_unary<ReciprocalOp>(t, DPB_U_RECIPROCAL);
    reg_unary<FloorOp>(t, DPB_U_FLOOR);
    reg_unary<CeilOp>(t, DPB_U_CEIL);
    reg_unary<SignOp>(t, DPB_U_SIGN);
}
}  // namespace dpb
