// Type-independent planning of a reduction over trailing axes.
#pragma once

#include <stdint.h>

#include "ew_plan.h"

namespace dpb {

enum RedKind { RED_INNER = 0, RED_OUTER, RED_GENERIC };

struct RedPlan {
    int kind = RED_GENERIC;
    int64_t niter = 0;  // number of results
    int64_t nred = 0;   // elements reduced into each result
    // iteration (result) dimensions: extents, source strides, result strides
    int iter_nd = 0;
    int64_t iter_shape[kMaxD];
    int64_t iter_src[kMaxD];
    int64_t iter_dst[kMaxD];
    // reduction dimensions: extents and source strides
    int red_nd = 0;
    int64_t red_shape[kMaxD];
    int64_t red_src[kMaxD];
    int64_t src_offset = 0;  // element displacement of the source base
    int64_t dst_offset = 0;  // element displacement of the result base
};

// Plan from explicit iteration/reduction dimensions (strides in elements).
// `keep_order` keeps the C order of the reduction dimensions (needed when the
// position inside the reduced sub-space is part of the result).
int make_red_plan(int iter_nd, const int64_t *iter_shape, const int64_t *iter_src,
                  const int64_t *iter_dst, int red_nd, const int64_t *red_shape,
                  const int64_t *red_src, bool keep_order, RedPlan &plan);

}  // namespace dpb
