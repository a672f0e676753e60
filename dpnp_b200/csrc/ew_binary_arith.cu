// add, subtract, multiply, true_divide.
#include "ew_register.cuh"
namespace dpb {
void register_binary_arith(EwTables &t)
{
    reg_binary<AddOp>(t, DPB_B_ADD);
    reg_binary<SubtractOp>(t, DPB_B_SUBTRACT);
    reg_binary<MultiplyOp>(t, DPB_B_MULTIPLY);
    reg_binary<TrueDivideOp>(t, DPB_B_TRUE_DIVIDE);
}
}  // namespace dpb
