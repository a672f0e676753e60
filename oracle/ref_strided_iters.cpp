// TEST INFRASTRUCTURE, not product code.
//
// extern "C" wrappers around the iteration-space simplifier of the reference,
// compiled against the reference's own header where it lies:
//   dpnp/tensor/libtensor/include/utils/strided_iters.hpp:363-983
// (simplify_iteration_stride, _two_strides, _three_strides, _four_strides,
// compact_iteration).  The header is free of SYCL, so g++ alone builds it.
// Only the build recipe in this directory passes the include path; nothing of
// the reference is copied here.  The resulting library (oracle/_ref/) is used
// by the tests to pin dpb_simplify_iteration_space against the reference.
#include <cstdint>

#include "utils/strided_iters.hpp"

namespace rs = dpnp::tensor::strides;

extern "C" {

// strides: narrays*nd values laid out [array][dim]; offsets: narrays outputs.
// Returns the collapsed number of dimensions; shape and strides are rewritten
// in place with row length `nd` kept for the strides.
int ref_simplify(int narrays, int nd, int64_t *shape, int64_t *strides, int64_t *offsets)
{
    int64_t d1 = 0, d2 = 0, d3 = 0, d4 = 0;
    int m = nd;
    switch (narrays) {
    case 1:
        m = rs::simplify_iteration_stride(nd, shape, strides, d1);
        break;
    case 2:
        m = rs::simplify_iteration_two_strides(nd, shape, strides, strides + nd, d1, d2);
        break;
    case 3:
        m = rs::simplify_iteration_three_strides(nd, shape, strides, strides + nd, strides + 2 * nd, d1,
                                                 d2, d3);
        break;
    case 4:
        m = rs::simplify_iteration_four_strides(nd, shape, strides, strides + nd, strides + 2 * nd,
                                                strides + 3 * nd, d1, d2, d3, d4);
        break;
    default:
        return -1;
    }
    offsets[0] = d1;
    if (narrays > 1) offsets[1] = d2;
    if (narrays > 2) offsets[2] = d3;
    if (narrays > 3) offsets[3] = d4;
    return m;
}

int ref_compact(int nd, int64_t *shape, int64_t *strides)
{
    return rs::compact_iteration(nd, shape, strides);
}

}  // extern "C"
