// Reduction entry points of the C ABI.  The dispatch-level functions follow
// the argument checks of py_reduction_over_axis and py_search_over_axis
// (dpnp/tensor/libtensor/source/reductions/reduction_over_axis.hpp:173-501,780-1047).
#include <mutex>
#include <vector>

#include "iterspace.h"
#include "reduce_register.cuh"

namespace dpb {

static RedTables g_red;
static std::once_flag g_red_once;

const RedTables &red_tables()
{
    std::call_once(g_red_once, [] {
        register_reduce_sum(g_red);
        register_reduce_prod(g_red);
        register_reduce_minmax(g_red);
        register_reduce_search(g_red);
        register_reduce_fp(g_red);
    });
    return g_red;
}

static inline bool valid_type(int t) { return t >= 0 && t < DPB_NUM_TYPES; }

static int lookup(bool search, int op, int t_in, int t_out, red_fn_t &fn)
{
    if (!valid_type(t_in) || !valid_type(t_out)) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (search) {
        if (op < 0 || op >= DPB_S_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown search op %d", op);
        fn = (t_out == DPB_INT64) ? red_tables().search[op][t_in] : nullptr;
    }
    else {
        if (op < 0 || op >= DPB_R_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown reduction op %d", op);
        fn = red_tables().reduce[op][t_in][t_out];
    }
    if (!fn) return set_error(DPB_ERR_RUNTIME, "Datatypes are not supported");
    return DPB_OK;
}

static int run_plan(red_fn_t fn, const RedPlan &plan, const void *arg, int t_in, void *res, int t_out,
                    void *stream)
{
    const char *a = static_cast<const char *>(arg) + plan.src_offset * type_size(t_in);
    char *r = static_cast<char *>(res) + plan.dst_offset * type_size(t_out);
    return fn(plan, a, r, static_cast<cudaStream_t>(stream));
}

static int contig_axis1(bool search, int op, int t_in, int t_out, int64_t iter_nelems,
                        int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                        int64_t res_off, void *stream)
{
    red_fn_t fn;
    DPB_TRY(lookup(search, op, t_in, t_out, fn));
    if (iter_nelems < 0 || reduction_nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    const int64_t ish = iter_nelems, isrc = reduction_nelems, idst = 1;
    const int64_t rsh = reduction_nelems, rsrc = 1;
    RedPlan plan;
    DPB_TRY(make_red_plan(1, &ish, &isrc, &idst, 1, &rsh, &rsrc, search, plan));
    plan.src_offset += arg_off;
    plan.dst_offset += res_off;
    return run_plan(fn, plan, arg, t_in, res, t_out, stream);
}

static int contig_axis0(bool search, int op, int t_in, int t_out, int64_t iter_nelems,
                        int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                        int64_t res_off, void *stream)
{
    red_fn_t fn;
    DPB_TRY(lookup(search, op, t_in, t_out, fn));
    if (iter_nelems < 0 || reduction_nelems < 0) return set_error(DPB_ERR_VALUE, "negative size");
    const int64_t ish = iter_nelems, isrc = 1, idst = 1;
    const int64_t rsh = reduction_nelems, rsrc = iter_nelems;
    RedPlan plan;
    DPB_TRY(make_red_plan(1, &ish, &isrc, &idst, 1, &rsh, &rsrc, search, plan));
    plan.src_offset += arg_off;
    plan.dst_offset += res_off;
    return run_plan(fn, plan, arg, t_in, res, t_out, stream);
}

static int strided(bool search, int op, int t_in, int t_out, const void *arg, void *res, int iter_nd,
                   const int64_t *iter_ss, int64_t iter_arg_off, int64_t iter_res_off, int red_nd,
                   const int64_t *red_ss, int64_t red_arg_off, void *stream)
{
    red_fn_t fn;
    DPB_TRY(lookup(search, op, t_in, t_out, fn));
    if (iter_nd < 0 || red_nd < 0 || iter_nd > DPB_MAX_ND || red_nd > DPB_MAX_ND ||
        (iter_nd > 0 && !iter_ss) || (red_nd > 0 && !red_ss))
        return set_error(DPB_ERR_VALUE, "bad shape/stride arguments");
    RedPlan plan;
    DPB_TRY(make_red_plan(iter_nd, iter_ss, iter_ss + iter_nd, iter_ss + 2 * iter_nd, red_nd, red_ss,
                          red_ss + red_nd, search, plan));
    plan.src_offset += iter_arg_off + red_arg_off;
    plan.dst_offset += iter_res_off;
    return run_plan(fn, plan, arg, t_in, res, t_out, stream);
}

// Shared body of dpb_reduction_over_axis and dpb_search_over_axis.
static int over_axis(bool search, int op, const dpb_array *src, int k, const dpb_array *dst,
                     void *stream)
{
    DPB_TRY(check_array(src, "src"));
    DPB_TRY(check_array(dst, "dst"));
    if (k <= 0) return set_error(DPB_ERR_VALUE, "Trailing_dim_to_reduce must be positive, but got %d", k);
    const int src_nd = src->nd;
    if (dst->nd + k != src_nd)
        return set_error(DPB_ERR_VALUE,
                         "Destination array rank does not match input array rank and number of "
                         "reduced dimensions");
    const int iter_nd = dst->nd;
    for (int i = 0; i < iter_nd; ++i)
        if (src->shape[i] != dst->shape[i])
            return set_error(DPB_ERR_VALUE, "Destination shape does not match unreduced dimensions of the input shape");
    if (src->device != dst->device)
        return set_error(DPB_ERR_VALUE, "Execution queue is not compatible with allocation queues");
    if (!(dst->flags & DPB_FLAG_WRITABLE)) return set_error(DPB_ERR_VALUE, "output array is read-only.");
    int64_t dst_nelems = num_elements(*dst);
    if (dst_nelems == 0) return DPB_OK;
    {
        int64_t lo, hi;
        displacement_range(*dst, lo, hi);
        if (hi - lo + 1 < dst_nelems)
            return set_error(DPB_ERR_VALUE,
                             "Memory addressed by the output array is not sufficiently ample.");
    }
    if (arrays_overlap(*src, *dst))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    red_fn_t fn;
    DPB_TRY(lookup(search, op, src->typenum, dst->typenum, fn));

    std::vector<int64_t> ss = strides_of(*src), ds = strides_of(*dst);
    RedPlan plan;
    DPB_TRY(make_red_plan(iter_nd, src->shape, ss.data(), ds.data(), k, src->shape + iter_nd,
                          ss.data() + iter_nd, search, plan));
    return run_plan(fn, plan, src->data, src->typenum, dst->data, dst->typenum, stream);
}

}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_reduce_dtype_supported(int op, int t_in, int t_out)
{
    if (op < 0 || op >= DPB_R_NUM_OPS || !valid_type(t_in) || !valid_type(t_out)) return 0;
    return red_tables().reduce[op][t_in][t_out] != nullptr;
}

int dpb_reduce_axis1_contig(int op, int t_in, int t_out, int64_t iter_nelems,
                            int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                            int64_t res_off, void *stream)
{
    return contig_axis1(false, op, t_in, t_out, iter_nelems, reduction_nelems, arg, arg_off, res,
                        res_off, stream);
}

int dpb_reduce_axis0_contig(int op, int t_in, int t_out, int64_t iter_nelems,
                            int64_t reduction_nelems, const void *arg, int64_t arg_off, void *res,
                            int64_t res_off, void *stream)
{
    return contig_axis0(false, op, t_in, t_out, iter_nelems, reduction_nelems, arg, arg_off, res,
                        res_off, stream);
}

int dpb_reduce_strided(int op, int t_in, int t_out, int64_t iter_nelems, int64_t reduction_nelems,
                       const void *arg, void *res, int iter_nd, const int64_t *iter_shape_strides,
                       int64_t iter_arg_off, int64_t iter_res_off, int red_nd,
                       const int64_t *red_shape_strides, int64_t red_arg_off, void *stream)
{
    (void)iter_nelems;
    (void)reduction_nelems;
    return strided(false, op, t_in, t_out, arg, res, iter_nd, iter_shape_strides, iter_arg_off,
                   iter_res_off, red_nd, red_shape_strides, red_arg_off, stream);
}

int dpb_search_axis1_contig(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                            const void *arg, int64_t arg_off, void *res, int64_t res_off, void *stream)
{
    return contig_axis1(true, op, t_in, DPB_INT64, iter_nelems, reduction_nelems, arg, arg_off, res,
                        res_off, stream);
}

int dpb_search_axis0_contig(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                            const void *arg, int64_t arg_off, void *res, int64_t res_off, void *stream)
{
    return contig_axis0(true, op, t_in, DPB_INT64, iter_nelems, reduction_nelems, arg, arg_off, res,
                        res_off, stream);
}

int dpb_search_strided(int op, int t_in, int64_t iter_nelems, int64_t reduction_nelems,
                       const void *arg, void *res, int iter_nd, const int64_t *iter_shape_strides,
                       int64_t iter_arg_off, int64_t iter_res_off, int red_nd,
                       const int64_t *red_shape_strides, int64_t red_arg_off, void *stream)
{
    (void)iter_nelems;
    (void)reduction_nelems;
    return strided(true, op, t_in, DPB_INT64, arg, res, iter_nd, iter_shape_strides, iter_arg_off,
                   iter_res_off, red_nd, red_shape_strides, red_arg_off, stream);
}

int dpb_reduction_over_axis(int op, const dpb_array *src, int trailing_dims_to_reduce,
                            const dpb_array *dst, void *stream)
{
    return over_axis(false, op, src, trailing_dims_to_reduce, dst, stream);
}

int dpb_search_over_axis(int op, const dpb_array *src, int trailing_dims_to_reduce,
                         const dpb_array *dst, void *stream)
{
    return over_axis(true, op, src, trailing_dims_to_reduce, dst, stream);
}

}  // extern "C"
