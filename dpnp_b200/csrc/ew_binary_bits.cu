// bitwise and/or/xor and the shifts (bool and integer types).
#include "ew_register.cuh"
namespace dpb {
void register_binary_bits(EwTables &t)
{
    reg_binary<BitwiseAndOp>(t, DPB_B_BITWISE_AND);
    reg_binary<BitwiseOrOp>(t, DPB_B_BITWISE_OR);
    reg_binary<BitwiseXorOp>(t, DPB_B_BITWISE_XOR);
    reg_binary<LeftShiftOp>(t, DPB_B_BITWISE_LEFT_SHIFT);
    reg_binary<RightShiftOp>(t, DPB_B_BITWISE_RIGHT_SHIFT);
}
}  // namespace dpb
