// trunc, round, signbit, bitwise_invert and the complex-part functions.
#include "ew_register.cuh"
namespace dpb {
void register_unary_misc2(EwTables &t)
{
    reg_unary<TruncOp>(t, DPB_U_TRUNC);
    reg_unary<RoundOp>(t, DPB_U_ROUND);
    reg_unary<SignbitOp>(t, DPB_U_SIGNBIT);
    reg_unary<BitwiseInvertOp>(t, DPB_U_BITWISE_INVERT);
    reg_unary<ConjOp>(t, DPB_U_CONJ);
    reg_unary<RealOp>(t, DPB_U_REAL);
    reg_unary<ImagOp>(t, DPB_U_IMAG);
    reg_unary<AngleOp>(t, DPB_U_ANGLE);
    reg_unary<ProjOp>(t, DPB_U_PROJ);
}
}  // namespace dpb
