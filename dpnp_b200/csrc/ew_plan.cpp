// Planning of elementwise launches (see ew_plan.h).
//
// The contiguity tests and the fall-back order mirror what py_binary_ufunc does
// before it picks a kernel (dpnp/tensor/libtensor/source/elementwise_functions/
// elementwise_functions.hpp:383-553): contiguous operands first, then the
// collapsed iteration space, with extra specialisations the reference lacks
// (unit-stride rows with arbitrary outer strides; transposed operands).
#include "ew_plan.h"

#include <vector>

#include "common.cuh"
#include "iterspace.h"

namespace dpb {

int make_ew_plan(int narr, int nd, const int64_t *shape, const int64_t *strides,
                 const int *elem_sizes, EwPlan &plan)
{
    plan = EwPlan();
    plan.narr = narr;
    const int nin = narr - 1;
    const int out = narr - 1;
    int64_t n = 1;
    for (int i = 0; i < nd; ++i) n *= shape[i];
    plan.n = n;
    for (int k = 0; k < 4; ++k) plan.offsets[k] = 0;
    if (n == 0) {
        plan.kind = EW_CONTIG;
        plan.nd = 0;
        return DPB_OK;
    }

    // drop extent-1 dimensions, then collapse
    std::vector<int64_t> sh;
    std::vector<int64_t> st(static_cast<size_t>(narr) * (nd > 0 ? nd : 1));
    int m = 0;
    for (int i = 0; i < nd; ++i)
        if (shape[i] != 1) ++m;
    sh.resize(m > 0 ? m : 1);
    {
        int j = 0;
        for (int i = 0; i < nd; ++i) {
            if (shape[i] == 1) continue;
            sh[j] = shape[i];
            for (int k = 0; k < narr; ++k) st[k * m + j] = strides[k * nd + i];
            ++j;
        }
    }
    int64_t offs[kMaxArrays] = {0, 0, 0, 0};
    int cnd = (m > 0) ? simplify_iteration_space(narr, m, sh.data(), st.data(), offs) : 0;
    if (cnd > kMaxD)
        return set_error(DPB_ERR_RUNTIME,
                         "iteration space keeps %d dimensions after collapsing; at most %d are "
                         "supported", cnd, kMaxD);
    if (cnd == 0) {
        // single element
        cnd = 1;
        sh[0] = 1;
        st.assign(static_cast<size_t>(narr), 1);
    }
    plan.nd = cnd;
    for (int i = 0; i < cnd; ++i) {
        plan.shape[i] = sh[i];
        for (int k = 0; k < narr; ++k) plan.strides[k][i] = st[k * cnd + i];
    }
    for (int k = 0; k < narr; ++k) plan.offsets[k] = offs[k];

    if (tuning_force_generic()) {   // debugging aid: the kernel with no layout assumptions
        plan.kind = EW_GENERIC;
        return DPB_OK;
    }
    const int last = cnd - 1;
    // (1) one collapsed dimension, output dense, inputs dense or one element
    if (cnd == 1 && (plan.strides[out][0] == 1 || n == 1)) {
        bool ok = true;
        unsigned mask = 0;
        for (int k = 0; k < nin; ++k) {
            const int64_t s = plan.strides[k][0];
            if (s == 0 && n > 1) mask |= (1u << k);
            else if (s != 1 && n > 1) ok = false;
        }
        if (ok) {
            plan.kind = EW_CONTIG;
            plan.bcast_mask = mask;
            return DPB_OK;
        }
    }
    // the specialised strided kernels index rows/batches with 31-bit integers
    bool small_outer = true;
    {
        int64_t outer = 1;
        for (int i = 0; i < last; ++i) {
            outer *= plan.shape[i];
            if (outer >= (int64_t(1) << 31)) small_outer = false;
        }
    }
    // (2) rows: innermost dimension unit-stride (or broadcast) everywhere
    if (small_outer && plan.strides[out][last] == 1 && plan.shape[last] >= 8) {
        bool ok = true;
        for (int k = 0; k < nin; ++k) {
            const int64_t s = plan.strides[k][last];
            if (s != 0 && s != 1) ok = false;
        }
        if (ok) {
            plan.kind = EW_ROWS;
            return DPB_OK;
        }
    }
    // (3) transpose: output unit-stride along the last dimension, some input
    //     unit-stride along another dimension P instead
    if (small_outer && cnd >= 2 && plan.strides[out][last] == 1 && plan.shape[last] >= 8) {
        int pdim = -1;
        for (int k = 0; k < nin && pdim < 0; ++k) {
            const int64_t s = plan.strides[k][last];
            if (s == 0 || s == 1) continue;
            for (int d = 0; d < last; ++d)
                if (plan.strides[k][d] == 1 && plan.shape[d] >= 8) {
                    pdim = d;
                    break;
                }
        }
        if (pdim >= 0) {
            unsigned staged = 0;
            for (int k = 0; k < nin; ++k) {
                const int64_t s = plan.strides[k][last];
                if (s != 0 && s != 1 && plan.strides[k][pdim] == 1 && elem_sizes[k] <= 8)
                    staged |= (1u << k);
            }
            if (staged) {
                plan.kind = EW_TRANSPOSE;
                plan.tdim = pdim;
                plan.staged_mask = staged;
                return DPB_OK;
            }
        }
    }
    plan.kind = EW_GENERIC;
    return DPB_OK;
}

}  // namespace dpb
