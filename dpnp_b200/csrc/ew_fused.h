// What the two executors of a fused program share: the interpreter (ew_fused.cu) and the
// specialised kernels compiled at run time (ew_fused_jit.cu).
#pragma once

#include <stdint.h>

#include "../../include/dpnp_b200.h"

namespace dpb {

constexpr int kFusedMaxInstr = 192;
constexpr int kFusedMaxImm = 48;
constexpr int kFusedMaxIn = 12;
constexpr int kFusedMaxOut = 8;
constexpr int kFusedMaxReg = 24;

// operand encoding (8 bits)
constexpr unsigned kOpndImm = 64;      // 64 + i: immediate i
constexpr unsigned kOpndIn = 128;      // 128 + i: input array i, read where it is used
constexpr unsigned kOpndAcc = 255;     // result of the previous instruction
constexpr unsigned kNoDst = 255;       // result stays in the accumulator only

// Limits, pointers and every index of every instruction; `aligned` (may be null) reports
// whether all array pointers allow 16-byte accesses.
int fused_check_program(const dpb_fused_program *prog, int64_t n, bool *aligned);

}  // namespace dpb
