// Unary transcendental operations.
#include "ew_register.cuh"
#include "ew_erf.cuh"
namespace dpb {
void register_unary_math(EwTables &t)
{
    reg_unary<ExpOp>(t, DPB_U_EXP);
    reg_unary<LogOp>(t, DPB_U_LOG);
    reg_unary<SqrtOp>(t, DPB_U_SQRT);
    reg_unary<ErfOp>(t, DPB_U_ERF);
    reg_unary<SinOp>(t, DPB_U_SIN);
    reg_unary<CosOp>(t, DPB_U_COS);
    reg_unary<TanhOp>(t, DPB_U_TANH);
    reg_unary<Expm1Op>(t, DPB_U_EXPM1);
    reg_unary<Log1pOp>(t, DPB_U_LOG1P);
}
}  // namespace dpb
