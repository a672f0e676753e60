// atan2, hypot, copysign, logaddexp, nextafter (floating types only).
#include "ew_register.cuh"
namespace dpb {
void register_binary_fp2(EwTables &t)
{
    reg_binary<Atan2Op>(t, DPB_B_ATAN2);
    reg_binary<HypotOp>(t, DPB_B_HYPOT);
    reg_binary<CopysignOp>(t, DPB_B_COPYSIGN);
    reg_binary<LogaddexpOp>(t, DPB_B_LOGADDEXP);
    reg_binary<NextafterOp>(t, DPB_B_NEXTAFTER);
}
}  // namespace dpb
