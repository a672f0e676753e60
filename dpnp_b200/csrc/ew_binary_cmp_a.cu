// equal, not_equal, less.
#include "ew_register.cuh"
namespace dpb {
void register_binary_cmp_a(EwTables &t)
{
    reg_binary<EqualOp>(t, DPB_B_EQUAL);
    reg_binary<NotEqualOp>(t, DPB_B_NOT_EQUAL);
    reg_binary<LessOp>(t, DPB_B_LESS);
}
}  // namespace dpb
