// Type-independent planning of an elementwise launch: collapse the iteration
// space of all operands and pick the kernel family.
#pragma once

#include <stdint.h>

#include "../../include/dpnp_b200.h"

namespace dpb {

constexpr int kMaxD = DPB_MAX_COLLAPSED_ND;

enum EwKind { EW_CONTIG = 0, EW_ROWS, EW_TRANSPOSE, EW_GENERIC };

// Arrays are ordered inputs first, output last (narr = inputs + 1).
struct EwPlan {
    int narr = 0;
    int kind = EW_GENERIC;
    int nd = 0;
    int64_t n = 0;                 // number of output elements
    int64_t shape[kMaxD];
    int64_t strides[4][kMaxD];     // [array][dim], elements
    int64_t offsets[4];            // element displacement of each base pointer
    unsigned bcast_mask = 0;       // EW_CONTIG: inputs that are a single element
    int tdim = -1;                 // EW_TRANSPOSE: dimension P
    unsigned staged_mask = 0;      // EW_TRANSPOSE: inputs staged through shared memory
};

// Build a plan from raw shape/strides ([array][dim], narr*nd values).
// `elem_sizes` are bytes per element of each array.  Fails with DPB_ERR_RUNTIME
// if more than kMaxD dimensions remain after collapsing.
int make_ew_plan(int narr, int nd, const int64_t *shape, const int64_t *strides,
                 const int *elem_sizes, EwPlan &plan);

}  // namespace dpb
