// Host-side iteration-space algebra (see iterspace.h).
//
// Behavioural spec: dpnp/tensor/libtensor/include/utils/strided_iters.hpp:363-983
// (simplify_iteration_* and compact_iteration), source/simplify_iteration_space.cpp:51-264
// and include/utils/memory_overlap.hpp:52-151 of the reference.
#include "iterspace.h"

#include <algorithm>
#include <cstdlib>
#include <numeric>

#include "common.cuh"

namespace dpb {

static inline int64_t iabs(int64_t v) { return v < 0 ? -v : v; }

int simplify_iteration_space(int narrays, int nd, int64_t *shape, int64_t *strides,
                             int64_t *offsets)
{
    for (int a = 0; a < narrays; ++a) offsets[a] = 0;
    if (nd < 1) return nd;

    auto st = [&](int a, int d) -> int64_t & { return strides[a * nd + d]; };

    // 1. order dimensions by decreasing |stride|; the last array decides first,
    //    then the one before it, ..., finally larger extents first.
    std::vector<int> order(nd);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) {
        for (int a = narrays - 1; a >= 0; --a) {
            int64_t sx = iabs(st(a, x)), sy = iabs(st(a, y));
            if (sx != sy) return sx > sy;
        }
        return shape[x] > shape[y];
    });

    std::vector<int64_t> sh(nd);
    std::vector<int64_t> sr(static_cast<size_t>(narrays) * nd);
    bool mergeable = true;
    for (int i = 0; i < nd; ++i) {
        int p = order[i];
        sh[i] = shape[p];
        // 2. a dimension walked backwards by every array that moves along it
        //    is reversed; the base offsets absorb the shift.
        bool none_positive = true, some_negative = false;
        for (int a = 0; a < narrays; ++a) {
            none_positive = none_positive && st(a, p) <= 0;
            some_negative = some_negative || st(a, p) < 0;
        }
        bool flip = none_positive && some_negative;
        for (int a = 0; a < narrays; ++a) {
            int64_t s = st(a, p);
            if (flip) {
                offsets[a] += s * (sh[i] - 1);
                s = -s;
            }
            if (s < 0) mergeable = false;
            sr[a * nd + i] = s;
        }
    }

    // 3. merge neighbours (i, i+1) when stepping past the end of dimension
    //    i+1 lands exactly on the next element of dimension i in every array.
    int m = nd;
    if (mergeable) {
        int i = 0;
        while (i + 1 < m) {
            bool chain = true;
            for (int a = 0; a < narrays && chain; ++a) {
                chain = sr[a * nd + i] == sh[i + 1] * sr[a * nd + i + 1];
            }
            if (chain) {
                sh[i] *= sh[i + 1];
                for (int a = 0; a < narrays; ++a) {
                    sr[a * nd + i] = sr[a * nd + i + 1];
                    for (int k = i + 1; k + 1 < m; ++k) sr[a * nd + k] = sr[a * nd + k + 1];
                }
                for (int k = i + 1; k + 1 < m; ++k) sh[k] = sh[k + 1];
                --m;
                // a merge can enable a merge with the previous dimension
                if (i > 0) --i;
            }
            else {
                ++i;
            }
        }
    }

    for (int i = 0; i < m; ++i) shape[i] = sh[i];
    // repack strides with the new row length m, in place: destination index
    // a*m+i never exceeds source index a*nd+i, so a forward copy is safe
    for (int a = 0; a < narrays; ++a)
        for (int i = 0; i < m; ++i) strides[a * m + i] = sr[a * nd + i];
    return m;
}

int compact_iteration(int nd, int64_t *shape, int64_t *strides)
{
    if (nd < 2) return nd;
    for (int i = 0; i < nd; ++i)
        if (strides[i] < 0) return nd;
    int m = nd;
    int i = 0;
    while (i + 1 < m) {
        if (strides[i] == shape[i + 1] * strides[i + 1]) {
            shape[i] *= shape[i + 1];
            strides[i] = strides[i + 1];
            for (int k = i + 1; k + 1 < m; ++k) {
                shape[k] = shape[k + 1];
                strides[k] = strides[k + 1];
            }
            --m;
            if (i > 0) --i;
        }
        else {
            ++i;
        }
    }
    return m;
}

std::vector<int64_t> strides_of(const dpb_array &a)
{
    std::vector<int64_t> s(a.nd);
    if (a.strides) {
        for (int i = 0; i < a.nd; ++i) s[i] = a.strides[i];
    }
    else {
        int64_t acc = 1;
        for (int i = a.nd - 1; i >= 0; --i) {
            s[i] = acc;
            acc *= a.shape[i];
        }
    }
    return s;
}

int64_t num_elements(const dpb_array &a)
{
    int64_t n = 1;
    for (int i = 0; i < a.nd; ++i) n *= a.shape[i];
    return n;
}

void displacement_range(const dpb_array &a, int64_t &lo, int64_t &hi)
{
    lo = 0;
    hi = 0;
    if (num_elements(a) == 0) return;
    std::vector<int64_t> s = strides_of(a);
    for (int i = 0; i < a.nd; ++i) {
        int64_t span = s[i] * (a.shape[i] - 1);
        if (span < 0) lo += span;
        else hi += span;
    }
}

bool arrays_overlap(const dpb_array &a, const dpb_array &b)
{
    if (num_elements(a) == 0 || num_elements(b) == 0) return false;
    int64_t alo, ahi, blo, bhi;
    displacement_range(a, alo, ahi);
    displacement_range(b, blo, bhi);
    const int64_t asz = type_size(a.typenum), bsz = type_size(b.typenum);
    const char *ap = static_cast<const char *>(a.data);
    const char *bp = static_cast<const char *>(b.data);
    const char *a0 = ap + alo * asz, *a1 = ap + (ahi + 1) * asz;  // [a0, a1)
    const char *b0 = bp + blo * bsz, *b1 = bp + (bhi + 1) * bsz;
    return a0 < b1 && b0 < a1;
}

bool same_logical_tensors(const dpb_array &a, const dpb_array &b)
{
    if (a.data != b.data || a.typenum != b.typenum || a.nd != b.nd) return false;
    for (int i = 0; i < a.nd; ++i)
        if (a.shape[i] != b.shape[i]) return false;
    std::vector<int64_t> sa = strides_of(a), sb = strides_of(b);
    return sa == sb;
}

int check_array(const dpb_array *a, const char *what)
{
    if (!a) return set_error(DPB_ERR_VALUE, "%s: null array descriptor", what);
    if (a->nd < 0 || a->nd > DPB_MAX_ND)
        return set_error(DPB_ERR_VALUE, "%s: number of dimensions %d out of range", what, a->nd);
    if (a->typenum < 0 || a->typenum >= DPB_NUM_TYPES)
        return set_error(DPB_ERR_VALUE, "%s: unknown type id %d", what, a->typenum);
    if (a->nd > 0 && !a->shape) return set_error(DPB_ERR_VALUE, "%s: null shape", what);
    for (int i = 0; i < a->nd; ++i)
        if (a->shape[i] < 0) return set_error(DPB_ERR_VALUE, "%s: negative extent", what);
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_simplify_iteration_space(int narrays, int nd, int64_t *shape, int64_t *strides,
                                 int64_t *offsets, int *nd_out)
{
    if (narrays < 1 || narrays > kMaxArrays)
        return set_error(DPB_ERR_VALUE, "narrays must be 1..%d", kMaxArrays);
    if (nd < 0 || !nd_out || (nd > 0 && (!shape || !strides)) || !offsets)
        return set_error(DPB_ERR_VALUE, "dpb_simplify_iteration_space: bad arguments");
    *nd_out = simplify_iteration_space(narrays, nd, shape, strides, offsets);
    return DPB_OK;
}

int dpb_compact_iteration(int nd, int64_t *shape, int64_t *strides, int *nd_out)
{
    if (nd < 0 || !nd_out || (nd > 0 && (!shape || !strides)))
        return set_error(DPB_ERR_VALUE, "dpb_compact_iteration: bad arguments");
    *nd_out = compact_iteration(nd, shape, strides);
    return DPB_OK;
}

int dpb_array_overlap(const dpb_array *a, const dpb_array *b, int *overlap)
{
    DPB_TRY(check_array(a, "dpb_array_overlap"));
    DPB_TRY(check_array(b, "dpb_array_overlap"));
    *overlap = arrays_overlap(*a, *b) ? 1 : 0;
    return DPB_OK;
}

int dpb_same_logical_tensors(const dpb_array *a, const dpb_array *b, int *same)
{
    DPB_TRY(check_array(a, "dpb_same_logical_tensors"));
    DPB_TRY(check_array(b, "dpb_same_logical_tensors"));
    *same = same_logical_tensors(*a, *b) ? 1 : 0;
    return DPB_OK;
}

}  // extern "C"
