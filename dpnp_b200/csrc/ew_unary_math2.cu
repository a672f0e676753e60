// Inverse trigonometric, hyperbolic and base-2/10 functions, cbrt, rsqrt.
#include "ew_register.cuh"
namespace dpb {
void register_unary_math2(EwTables &t)
{
    reg_unary<AcosOp>(t, DPB_U_ACOS);
    reg_unary<AcoshOp>(t, DPB_U_ACOSH);
    reg_unary<AsinOp>(t, DPB_U_ASIN);
    reg_unary<AsinhOp>(t, DPB_U_ASINH);
    reg_unary<AtanOp>(t, DPB_U_ATAN);
    reg_unary<AtanhOp>(t, DPB_U_ATANH);
    reg_unary<CbrtOp>(t, DPB_U_CBRT);
    reg_unary<CoshOp>(t, DPB_U_COSH);
    reg_unary<SinhOp>(t, DPB_U_SINH);
    reg_unary<TanOp>(t, DPB_U_TAN);
    reg_unary<Exp2Op>(t, DPB_U_EXP2);
    reg_unary<Log2Op>(t, DPB_U_LOG2);
    reg_unary<Log10Op>(t, DPB_U_LOG10);
    reg_unary<RsqrtOp>(t, DPB_U_RSQRT);
}
}  // namespace dpb
