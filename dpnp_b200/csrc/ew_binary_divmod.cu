// floor_divide, remainder, logical_xor.
#include "ew_register.cuh"
namespace dpb {
void register_binary_divmod(EwTables &t)
{
    reg_binary<FloorDivideOp>(t, DPB_B_FLOOR_DIVIDE);
    reg_binary<RemainderOp>(t, DPB_B_REMAINDER);
    reg_binary<LogicalXorOp>(t, DPB_B_LOGICAL_XOR);
}
}  // namespace dpb
