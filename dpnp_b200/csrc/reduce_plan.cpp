// Planning of reductions (see reduce_plan.h).  The choice of kernel shape
// plays the role of the contiguity tests in py_reduction_over_axis
// (dpnp/tensor/libtensor/source/reductions/reduction_over_axis.hpp:259-442):
// iteration and reduction dimensions are collapsed separately, then
//   - a single unit-stride reduction dimension selects the inner kernel
//     (rows may sit anywhere: the iteration offsets are arbitrary),
//   - a unit-stride innermost iteration dimension selects the outer kernel,
//   - anything else takes the generic kernel.
#include "reduce_plan.h"

#include <vector>

#include "common.cuh"
#include "iterspace.h"

namespace dpb {

int make_red_plan(int iter_nd, const int64_t *iter_shape, const int64_t *iter_src,
                  const int64_t *iter_dst, int red_nd, const int64_t *red_shape,
                  const int64_t *red_src, bool keep_order, RedPlan &plan)
{
    plan = RedPlan();
    int64_t niter = 1, nred = 1;
    for (int i = 0; i < iter_nd; ++i) niter *= iter_shape[i];
    for (int i = 0; i < red_nd; ++i) nred *= red_shape[i];
    plan.niter = niter;
    plan.nred = nred;
    if (niter == 0) return DPB_OK;

    // iteration side: drop extent-1 dimensions, collapse (source, result) together
    {
        std::vector<int64_t> sh, st;
        int m = 0;
        for (int i = 0; i < iter_nd; ++i)
            if (iter_shape[i] != 1) ++m;
        sh.resize(m > 0 ? m : 1);
        st.resize(m > 0 ? 2 * m : 2);
        int j = 0;
        for (int i = 0; i < iter_nd; ++i) {
            if (iter_shape[i] == 1) continue;
            sh[j] = iter_shape[i];
            st[j] = iter_src[i];
            st[m + j] = iter_dst[i];
            ++j;
        }
        int64_t offs[kMaxArrays] = {0, 0, 0, 0};
        int c = m > 0 ? simplify_iteration_space(2, m, sh.data(), st.data(), offs) : 0;
        if (c > kMaxD)
            return set_error(DPB_ERR_RUNTIME, "too many iteration dimensions after collapsing (%d)", c);
        plan.iter_nd = c;
        for (int i = 0; i < c; ++i) {
            plan.iter_shape[i] = sh[i];
            plan.iter_src[i] = st[i];
            plan.iter_dst[i] = st[c + i];
        }
        plan.src_offset += offs[0];
        plan.dst_offset += offs[1];
    }
    // reduction side
    if (nred > 0) {
        std::vector<int64_t> sh, st;
        for (int i = 0; i < red_nd; ++i) {
            if (red_shape[i] == 1) continue;
            sh.push_back(red_shape[i]);
            st.push_back(red_src[i]);
        }
        int m = static_cast<int>(sh.size());
        int c = m;
        if (m > 0) {
            if (keep_order) {
                c = compact_iteration(m, sh.data(), st.data());
            }
            else {
                int64_t off = 0;
                c = simplify_iteration_space(1, m, sh.data(), st.data(), &off);
                plan.src_offset += off;
            }
        }
        if (c > kMaxD)
            return set_error(DPB_ERR_RUNTIME, "too many reduction dimensions after collapsing (%d)", c);
        plan.red_nd = c;
        for (int i = 0; i < c; ++i) {
            plan.red_shape[i] = sh[i];
            plan.red_src[i] = st[i];
        }
    }

    if (nred == 0) return DPB_OK;
    if (tuning_force_generic() && plan.iter_nd + plan.red_nd <= kMaxD) {
        plan.kind = RED_GENERIC;
        return DPB_OK;
    }
    const bool outer_ok = plan.iter_nd >= 1 && plan.iter_src[plan.iter_nd - 1] == 1 &&
                          plan.iter_dst[plan.iter_nd - 1] == 1 && plan.iter_shape[plan.iter_nd - 1] >= 16;
    if (plan.red_nd == 0 || (plan.red_nd == 1 && plan.red_src[0] == 1)) {
        plan.kind = RED_INNER;
    }
    else if (outer_ok) {
        plan.kind = RED_OUTER;
    }
    else if (plan.red_src[plan.red_nd - 1] == 1 && plan.red_shape[plan.red_nd - 1] >= 32 &&
             plan.iter_nd + plan.red_nd - 1 <= kMaxD) {
        // several reduction dimensions, the innermost unit-stride: rows of the inner kernel,
        // one per (result, outer reduction index)
        plan.kind = RED_INNER;
    }
    else {
        plan.kind = RED_GENERIC;
    }
    return DPB_OK;
}

}  // namespace dpb
