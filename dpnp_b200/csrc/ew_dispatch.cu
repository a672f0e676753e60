// Elementwise entry points of the C ABI: table lookup, argument validation and
// kernel selection.  The dispatch-level functions follow the checks and the
// error messages of the reference dispatchers py_unary_ufunc, py_binary_ufunc,
// py_binary_inplace_ufunc (dpnp/tensor/libtensor/source/elementwise_functions/
// elementwise_functions.hpp:76-251,305-563,611-804), py_where (source/where.cpp:73-245)
// and copy_usm_ndarray_into_usm_ndarray (source/copy_and_cast_usm_to_usm.cpp:76-...).
#include <cstring>
#include <mutex>
#include <vector>

#include "ew_register.cuh"
#include "iterspace.h"

namespace dpb {

static EwTables g_tables;
static std::once_flag g_tables_once;

const EwTables &ew_tables()
{
    std::call_once(g_tables_once, [] {
        register_unary_arith(g_tables);
        register_unary_math(g_tables);
        register_unary_pred(g_tables);
        register_binary_arith(g_tables);
        register_binary_misc(g_tables);
        register_binary_cmp_a(g_tables);
        register_binary_cmp_b(g_tables);
        register_unary_math2(g_tables);
        register_unary_misc2(g_tables);
        register_binary_fp2(g_tables);
        register_binary_bits(g_tables);
        register_binary_divmod(g_tables);
        register_where(g_tables);
        register_cast_a(g_tables);
        register_cast_b(g_tables);
    });
    return g_tables;
}

static inline bool valid_type(int t) { return t >= 0 && t < DPB_NUM_TYPES; }

static inline const char *byte_ptr(const void *p, int64_t off, int tn)
{
    return static_cast<const char *>(p) + off * type_size(tn);
}

// Plan from a host [shape | strides...] block as used by the kernel-level ABI.
static int plan_from_packed(int narr, int nd, const int64_t *shape_strides, const int *sizes,
                            EwPlan &plan)
{
    if (nd < 0 || nd > DPB_MAX_ND) return set_error(DPB_ERR_VALUE, "nd out of range");
    if (nd > 0 && !shape_strides) return set_error(DPB_ERR_VALUE, "null shape_strides");
    return make_ew_plan(narr, nd, shape_strides, shape_strides + nd, sizes, plan);
}

static int contig_plan(int narr, int64_t n, EwPlan &plan)
{
    plan = EwPlan();
    plan.narr = narr;
    plan.kind = EW_CONTIG;
    plan.nd = 1;
    plan.n = n;
    plan.shape[0] = n;
    for (int k = 0; k < 4; ++k) {
        plan.strides[k][0] = 1;
        plan.offsets[k] = 0;
    }
    return DPB_OK;
}

static int run(ew_fn_t fn, const EwPlan &plan, const void *const *in, const int *in_types, int nin,
               void *out, int out_type, void *stream)
{
    const void *pin[3] = {nullptr, nullptr, nullptr};
    for (int k = 0; k < nin; ++k) pin[k] = byte_ptr(in[k], plan.offsets[k], in_types[k]);
    void *pout = const_cast<char *>(byte_ptr(out, plan.offsets[nin], out_type));
    return fn(plan, pin, pout, static_cast<cudaStream_t>(stream));
}

static int lookup_unary(int op, int t_in, int t_out, ew_fn_t &fn)
{
    if (op < 0 || op >= DPB_U_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown unary op %d", op);
    if (!valid_type(t_in) || !valid_type(t_out)) return set_error(DPB_ERR_VALUE, "unknown type id");
    const EwEntry &e = ew_tables().unary[op][t_in];
    if (!e.fn)
        return set_error(DPB_ERR_RUNTIME, "Contiguous implementation is missing for src_typeid=%d",
                         t_in);
    if (e.rtype != t_out)
        return set_error(DPB_ERR_VALUE, "Destination array has unexpected elemental data type.");
    fn = e.fn;
    return DPB_OK;
}

static int lookup_binary(int op, int t_a, int t_b, int t_out, ew_fn_t &fn)
{
    if (op < 0 || op >= DPB_B_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown binary op %d", op);
    if (!valid_type(t_a) || !valid_type(t_b) || !valid_type(t_out))
        return set_error(DPB_ERR_VALUE, "unknown type id");
    const EwEntry &e = ew_tables().binary[op][t_a][t_b];
    if (!e.fn || e.rtype != t_out)
        return set_error(DPB_ERR_VALUE, "Destination array has unexpected elemental data type.");
    fn = e.fn;
    return DPB_OK;
}

static inline int size_class(int tn)
{
    switch (type_size(tn)) {
    case 1: return 0;
    case 2: return 1;
    case 4: return 2;
    case 8: return 3;
    default: return 4;
    }
}

// ------------------------------------------------ descriptor-level helpers

struct ArrView {
    const dpb_array *a;
    std::vector<int64_t> strides;
};

static int check_same_shape(const dpb_array *x, const dpb_array *dst)
{
    if (x->nd != dst->nd) return set_error(DPB_ERR_VALUE, "Array dimensions are not the same.");
    for (int i = 0; i < dst->nd; ++i)
        if (x->shape[i] != dst->shape[i])
            return set_error(DPB_ERR_VALUE, "Array shapes are not the same.");
    return DPB_OK;
}

static int check_writable(const dpb_array *dst)
{
    if (!(dst->flags & DPB_FLAG_WRITABLE))
        return set_error(DPB_ERR_VALUE, "output array is read-only.");
    return DPB_OK;
}

static int check_ample(const dpb_array *dst, int64_t nelems)
{
    int64_t lo, hi;
    displacement_range(*dst, lo, hi);
    if (hi - lo + 1 < nelems)
        return set_error(DPB_ERR_VALUE,
                         "Memory addressed by the output array is not sufficiently ample.");
    return DPB_OK;
}

static int check_device(std::initializer_list<const dpb_array *> arrs)
{
    int dev = -1;
    for (const dpb_array *a : arrs) {
        if (dev < 0) dev = a->device;
        else if (a->device != dev)
            return set_error(DPB_ERR_VALUE,
                             "Execution queue is not compatible with allocation queues");
    }
    return DPB_OK;
}

// Plan over descriptors: arrays ordered inputs first, output last.
static int plan_from_arrays(std::initializer_list<const dpb_array *> arrs, EwPlan &plan)
{
    const int narr = static_cast<int>(arrs.size());
    const dpb_array *dst = *(arrs.end() - 1);
    const int nd = dst->nd;
    std::vector<int64_t> st(static_cast<size_t>(narr) * (nd > 0 ? nd : 1));
    int sizes[4] = {1, 1, 1, 1};
    int k = 0;
    for (const dpb_array *a : arrs) {
        std::vector<int64_t> s = strides_of(*a);
        for (int i = 0; i < nd; ++i) st[k * nd + i] = s[i];
        sizes[k] = type_size(a->typenum);
        ++k;
    }
    return make_ew_plan(narr, nd, dst->shape, st.data(), sizes, plan);
}

}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_unary_result_type(int op, int t_in)
{
    if (op < 0 || op >= DPB_U_NUM_OPS || !valid_type(t_in)) return -1;
    return ew_tables().unary[op][t_in].rtype;
}

int dpb_binary_result_type(int op, int t_a, int t_b)
{
    if (op < 0 || op >= DPB_B_NUM_OPS || !valid_type(t_a) || !valid_type(t_b)) return -1;
    return ew_tables().binary[op][t_a][t_b].rtype;
}

// ------------------------------------------------------- kernel-level ABI

int dpb_unary_contig(int op, int t_in, int t_out, int64_t nelems, const void *in, int64_t in_off,
                     void *out, int64_t out_off, void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_unary(op, t_in, t_out, fn));
    if (nelems <= 0) return DPB_OK;
    EwPlan plan;
    contig_plan(2, nelems, plan);
    plan.offsets[0] = in_off;
    plan.offsets[1] = out_off;
    const void *ins[1] = {in};
    int types[1] = {t_in};
    return run(fn, plan, ins, types, 1, out, t_out, stream);
}

int dpb_unary_strided(int op, int t_in, int t_out, int64_t nelems, int nd,
                      const int64_t *shape_strides, const void *in, int64_t in_off, void *out,
                      int64_t out_off, void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_unary(op, t_in, t_out, fn));
    if (nelems <= 0) return DPB_OK;
    EwPlan plan;
    int sizes[4] = {type_size(t_in), type_size(t_out), 1, 1};
    DPB_TRY(plan_from_packed(2, nd, shape_strides, sizes, plan));
    plan.offsets[0] += in_off;
    plan.offsets[1] += out_off;
    const void *ins[1] = {in};
    int types[1] = {t_in};
    return run(fn, plan, ins, types, 1, out, t_out, stream);
}

int dpb_binary_contig(int op, int t_a, int t_b, int t_out, int64_t nelems, const void *a,
                      int64_t a_off, const void *b, int64_t b_off, void *out, int64_t out_off,
                      void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_binary(op, t_a, t_b, t_out, fn));
    if (nelems <= 0) return DPB_OK;
    EwPlan plan;
    contig_plan(3, nelems, plan);
    plan.offsets[0] = a_off;
    plan.offsets[1] = b_off;
    plan.offsets[2] = out_off;
    const void *ins[2] = {a, b};
    int types[2] = {t_a, t_b};
    return run(fn, plan, ins, types, 2, out, t_out, stream);
}

int dpb_binary_strided(int op, int t_a, int t_b, int t_out, int64_t nelems, int nd,
                       const int64_t *shape_strides, const void *a, int64_t a_off, const void *b,
                       int64_t b_off, void *out, int64_t out_off, void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_binary(op, t_a, t_b, t_out, fn));
    if (nelems <= 0) return DPB_OK;
    EwPlan plan;
    int sizes[4] = {type_size(t_a), type_size(t_b), type_size(t_out), 1};
    DPB_TRY(plan_from_packed(3, nd, shape_strides, sizes, plan));
    plan.offsets[0] += a_off;
    plan.offsets[1] += b_off;
    plan.offsets[2] += out_off;
    const void *ins[2] = {a, b};
    int types[2] = {t_a, t_b};
    return run(fn, plan, ins, types, 2, out, t_out, stream);
}

int dpb_binary_inplace_contig(int op, int t_rhs, int t_lhs, int64_t nelems, const void *rhs,
                              int64_t rhs_off, void *lhs, int64_t lhs_off, void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_binary(op, t_lhs, t_rhs, t_lhs, fn));
    if (nelems <= 0) return DPB_OK;
    EwPlan plan;
    contig_plan(3, nelems, plan);
    plan.offsets[0] = lhs_off;
    plan.offsets[1] = rhs_off;
    plan.offsets[2] = lhs_off;
    const void *ins[2] = {lhs, rhs};
    int types[2] = {t_lhs, t_rhs};
    return run(fn, plan, ins, types, 2, lhs, t_lhs, stream);
}

int dpb_binary_inplace_strided(int op, int t_rhs, int t_lhs, int64_t nelems, int nd,
                               const int64_t *shape_strides, const void *rhs, int64_t rhs_off,
                               void *lhs, int64_t lhs_off, void *stream)
{
    ew_fn_t fn;
    DPB_TRY(lookup_binary(op, t_lhs, t_rhs, t_lhs, fn));
    if (nelems <= 0) return DPB_OK;
    if (nd < 0 || nd > DPB_MAX_ND || (nd > 0 && !shape_strides))
        return set_error(DPB_ERR_VALUE, "bad shape_strides");
    // [shape | rhs | lhs] -> arrays (lhs, rhs, lhs)
    std::vector<int64_t> packed(static_cast<size_t>(4) * (nd > 0 ? nd : 1));
    for (int i = 0; i < nd; ++i) {
        packed[i] = shape_strides[i];
        packed[nd + i] = shape_strides[2 * nd + i];
        packed[2 * nd + i] = shape_strides[nd + i];
        packed[3 * nd + i] = shape_strides[2 * nd + i];
    }
    EwPlan plan;
    int sizes[4] = {type_size(t_lhs), type_size(t_rhs), type_size(t_lhs), 1};
    DPB_TRY(plan_from_packed(3, nd, packed.data(), sizes, plan));
    plan.offsets[0] += lhs_off;
    plan.offsets[1] += rhs_off;
    plan.offsets[2] += lhs_off;
    const void *ins[2] = {lhs, rhs};
    int types[2] = {t_lhs, t_rhs};
    return run(fn, plan, ins, types, 2, lhs, t_lhs, stream);
}

int dpb_where_contig(int t_cond, int t_val, int64_t nelems, const void *cond, const void *x1,
                     const void *x2, void *dst, void *stream)
{
    if (!valid_type(t_cond) || !valid_type(t_val)) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (nelems <= 0) return DPB_OK;
    ew_fn_t fn = ew_tables().where_[t_cond][size_class(t_val)];
    EwPlan plan;
    contig_plan(4, nelems, plan);
    const void *ins[3] = {cond, x1, x2};
    int types[3] = {t_cond, t_val, t_val};
    return run(fn, plan, ins, types, 3, dst, t_val, stream);
}

int dpb_where_strided(int t_cond, int t_val, int64_t nelems, int nd, const int64_t *shape_strides,
                      const void *cond, int64_t cond_off, const void *x1, int64_t x1_off,
                      const void *x2, int64_t x2_off, void *dst, int64_t dst_off, void *stream)
{
    if (!valid_type(t_cond) || !valid_type(t_val)) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (nelems <= 0) return DPB_OK;
    ew_fn_t fn = ew_tables().where_[t_cond][size_class(t_val)];
    EwPlan plan;
    int sizes[4] = {type_size(t_cond), type_size(t_val), type_size(t_val), type_size(t_val)};
    DPB_TRY(plan_from_packed(4, nd, shape_strides, sizes, plan));
    plan.offsets[0] += cond_off;
    plan.offsets[1] += x1_off;
    plan.offsets[2] += x2_off;
    plan.offsets[3] += dst_off;
    const void *ins[3] = {cond, x1, x2};
    int types[3] = {t_cond, t_val, t_val};
    return run(fn, plan, ins, types, 3, dst, t_val, stream);
}

int dpb_copy_cast_contig(int t_src, int t_dst, int64_t nelems, const void *src, int64_t src_off,
                         void *dst, int64_t dst_off, void *stream)
{
    if (!valid_type(t_src) || !valid_type(t_dst)) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (nelems <= 0) return DPB_OK;
    ew_fn_t fn = ew_tables().cast[t_src][t_dst];
    EwPlan plan;
    contig_plan(2, nelems, plan);
    plan.offsets[0] = src_off;
    plan.offsets[1] = dst_off;
    const void *ins[1] = {src};
    int types[1] = {t_src};
    return run(fn, plan, ins, types, 1, dst, t_dst, stream);
}

int dpb_copy_cast_strided(int t_src, int t_dst, int64_t nelems, int nd,
                          const int64_t *shape_strides, const void *src, int64_t src_off, void *dst,
                          int64_t dst_off, void *stream)
{
    if (!valid_type(t_src) || !valid_type(t_dst)) return set_error(DPB_ERR_VALUE, "unknown type id");
    if (nelems <= 0) return DPB_OK;
    ew_fn_t fn = ew_tables().cast[t_src][t_dst];
    EwPlan plan;
    int sizes[4] = {type_size(t_src), type_size(t_dst), 1, 1};
    DPB_TRY(plan_from_packed(2, nd, shape_strides, sizes, plan));
    plan.offsets[0] += src_off;
    plan.offsets[1] += dst_off;
    const void *ins[1] = {src};
    int types[1] = {t_src};
    return run(fn, plan, ins, types, 1, dst, t_dst, stream);
}

// ----------------------------------------------------- dispatch-level ABI

int dpb_unary_ufunc(int op, const dpb_array *src, const dpb_array *dst, void *stream)
{
    DPB_TRY(check_array(src, "src"));
    DPB_TRY(check_array(dst, "dst"));
    ew_fn_t fn;
    if (op < 0 || op >= DPB_U_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown unary op %d", op);
    {
        const EwEntry &e = ew_tables().unary[op][src->typenum];
        if (e.rtype != dst->typenum)
            return set_error(DPB_ERR_VALUE,
                             "Destination array has unexpected elemental data type.");
        fn = e.fn;
    }
    DPB_TRY(check_device({src, dst}));
    DPB_TRY(check_writable(dst));
    DPB_TRY(check_same_shape(src, dst));
    const int64_t n = num_elements(*src);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_ample(dst, n));
    if (arrays_overlap(*src, *dst) && !same_logical_tensors(*src, *dst))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    EwPlan plan;
    DPB_TRY(plan_from_arrays({src, dst}, plan));
    const void *ins[1] = {src->data};
    int types[1] = {src->typenum};
    return run(fn, plan, ins, types, 1, dst->data, dst->typenum, stream);
}

int dpb_binary_ufunc(int op, const dpb_array *src1, const dpb_array *src2, const dpb_array *dst,
                     void *stream)
{
    DPB_TRY(check_array(src1, "src1"));
    DPB_TRY(check_array(src2, "src2"));
    DPB_TRY(check_array(dst, "dst"));
    if (op < 0 || op >= DPB_B_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown binary op %d", op);
    const EwEntry &e = ew_tables().binary[op][src1->typenum][src2->typenum];
    if (e.rtype != dst->typenum || !e.fn)
        return set_error(DPB_ERR_VALUE, "Destination array has unexpected elemental data type.");
    DPB_TRY(check_device({src1, src2, dst}));
    DPB_TRY(check_writable(dst));
    DPB_TRY(check_same_shape(src1, dst));
    DPB_TRY(check_same_shape(src2, dst));
    const int64_t n = num_elements(*dst);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_ample(dst, n));
    if ((arrays_overlap(*src1, *dst) && !same_logical_tensors(*src1, *dst)) ||
        (arrays_overlap(*src2, *dst) && !same_logical_tensors(*src2, *dst)))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    EwPlan plan;
    DPB_TRY(plan_from_arrays({src1, src2, dst}, plan));
    const void *ins[2] = {src1->data, src2->data};
    int types[2] = {src1->typenum, src2->typenum};
    return run(e.fn, plan, ins, types, 2, dst->data, dst->typenum, stream);
}

int dpb_binary_inplace_ufunc(int op, const dpb_array *lhs, const dpb_array *rhs, void *stream)
{
    DPB_TRY(check_array(lhs, "lhs"));
    DPB_TRY(check_array(rhs, "rhs"));
    if (op < 0 || op >= DPB_B_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown binary op %d", op);
    DPB_TRY(check_writable(lhs));
    // the in-place form exists when op(lhs_type, rhs_type) yields lhs_type
    const EwEntry &e = ew_tables().binary[op][lhs->typenum][rhs->typenum];
    if (!e.fn || e.rtype != lhs->typenum)
        return set_error(DPB_ERR_VALUE, "Left-hand side array has unexpected elemental data type.");
    DPB_TRY(check_device({lhs, rhs}));
    DPB_TRY(check_same_shape(rhs, lhs));
    const int64_t n = num_elements(*lhs);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_ample(lhs, n));
    if (arrays_overlap(*rhs, *lhs) && !same_logical_tensors(*rhs, *lhs))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    EwPlan plan;
    DPB_TRY(plan_from_arrays({lhs, rhs, lhs}, plan));
    const void *ins[2] = {lhs->data, rhs->data};
    int types[2] = {lhs->typenum, rhs->typenum};
    return run(e.fn, plan, ins, types, 2, lhs->data, lhs->typenum, stream);
}

int dpb_where(const dpb_array *cond, const dpb_array *x1, const dpb_array *x2, const dpb_array *dst,
              void *stream)
{
    DPB_TRY(check_array(cond, "condition"));
    DPB_TRY(check_array(x1, "x1"));
    DPB_TRY(check_array(x2, "x2"));
    DPB_TRY(check_array(dst, "dst"));
    DPB_TRY(check_device({cond, x1, x2, dst}));
    DPB_TRY(check_writable(dst));
    if (x1->typenum != x2->typenum)
        return set_error(DPB_ERR_VALUE, "Value arrays must have the same data type");
    if (x1->typenum != dst->typenum)
        return set_error(DPB_ERR_VALUE, "Destination array has unexpected elemental data type.");
    if (cond->nd != dst->nd || x1->nd != dst->nd || x2->nd != dst->nd)
        return set_error(DPB_ERR_VALUE, "Array dimensions are not the same.");
    for (int i = 0; i < dst->nd; ++i)
        if (cond->shape[i] != dst->shape[i] || x1->shape[i] != dst->shape[i] ||
            x2->shape[i] != dst->shape[i])
            return set_error(DPB_ERR_VALUE, "Axes are not of matching shapes.");
    const int64_t n = num_elements(*dst);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_ample(dst, n));
    // the destination may coincide with an input exactly, never partially
    if ((arrays_overlap(*dst, *cond) && !same_logical_tensors(*dst, *cond)) ||
        (arrays_overlap(*dst, *x1) && !same_logical_tensors(*dst, *x1)) ||
        (arrays_overlap(*dst, *x2) && !same_logical_tensors(*dst, *x2)))
        return set_error(DPB_ERR_VALUE, "Destination array overlaps with input.");
    EwPlan plan;
    DPB_TRY(plan_from_arrays({cond, x1, x2, dst}, plan));
    ew_fn_t fn = ew_tables().where_[cond->typenum][size_class(dst->typenum)];
    const void *ins[3] = {cond->data, x1->data, x2->data};
    int types[3] = {cond->typenum, x1->typenum, x2->typenum};
    return run(fn, plan, ins, types, 3, dst->data, dst->typenum, stream);
}

int dpb_copy_array_into_array(const dpb_array *src, const dpb_array *dst, void *stream)
{
    DPB_TRY(check_array(src, "src"));
    DPB_TRY(check_array(dst, "dst"));
    DPB_TRY(check_same_shape(src, dst));
    const int64_t n = num_elements(*dst);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_writable(dst));
    DPB_TRY(check_device({src, dst}));
    DPB_TRY(check_ample(dst, n));
    if (same_logical_tensors(*src, *dst)) return DPB_OK;  // nothing to move
    if (arrays_overlap(*src, *dst))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    // identical types and both dense in the same order: one device memcpy
    const bool both_c = (src->flags & DPB_FLAG_C_CONTIGUOUS) && (dst->flags & DPB_FLAG_C_CONTIGUOUS);
    const bool both_f = (src->flags & DPB_FLAG_F_CONTIGUOUS) && (dst->flags & DPB_FLAG_F_CONTIGUOUS);
    if (src->typenum == dst->typenum && (both_c || both_f)) {
        note_copy("memcpy_d2d");
        return dpb_memcpy(dst->data, src->data, static_cast<size_t>(n) * type_size(src->typenum), 2,
                          stream);
    }
    EwPlan plan;
    DPB_TRY(plan_from_arrays({src, dst}, plan));
    ew_fn_t fn = ew_tables().cast[src->typenum][dst->typenum];
    const void *ins[1] = {src->data};
    int types[1] = {src->typenum};
    return run(fn, plan, ins, types, 1, dst->data, dst->typenum, stream);
}

int dpb_divide_by_scalar(const dpb_array *src, double scalar, const dpb_array *dst, void *stream)
{
    DPB_TRY(check_array(src, "src"));
    DPB_TRY(check_array(dst, "dst"));
    if (src->typenum != dst->typenum)
        return set_error(DPB_ERR_VALUE, "Destination array has unexpected elemental data type.");
    DPB_TRY(check_device({src, dst}));
    DPB_TRY(check_writable(dst));
    DPB_TRY(check_same_shape(src, dst));
    const int64_t n = num_elements(*dst);
    if (n == 0) return DPB_OK;
    DPB_TRY(check_ample(dst, n));
    if (arrays_overlap(*src, *dst) && !same_logical_tensors(*src, *dst))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    EwPlan plan;
    DPB_TRY(plan_from_arrays({src, dst}, plan));
    const void *pin[3] = {byte_ptr(src->data, plan.offsets[0], src->typenum), nullptr, nullptr};
    void *pout = const_cast<char *>(byte_ptr(dst->data, plan.offsets[1], dst->typenum));
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (src->typenum) {
    case DPB_HALF: {
        DivScalarF<half_t> f;
        f.s = static_cast<float>(scalar);
        return launch_ew(f, plan, pin, pout, s);
    }
    case DPB_FLOAT: {
        DivScalarF<float> f;
        f.s = static_cast<float>(scalar);
        return launch_ew(f, plan, pin, pout, s);
    }
    case DPB_DOUBLE: {
        DivScalarF<double> f;
        f.s = scalar;
        return launch_ew(f, plan, pin, pout, s);
    }
    default:
        return set_error(DPB_ERR_RUNTIME,
                         "divide_by_scalar is implemented for floating-point arrays only, got %s",
                         type_name(src->typenum));
    }
}

int dpb_full_array(const dpb_array *dst, const void *scalar_bits, void *stream)
{
    DPB_TRY(check_array(dst, "dst"));
    DPB_TRY(check_writable(dst));
    if (!scalar_bits) return set_error(DPB_ERR_VALUE, "null fill value");
    const int64_t n = num_elements(*dst);
    if (n == 0) return DPB_OK;
    // a fill is a 0-input elementwise op over the destination alone
    std::vector<int64_t> st = strides_of(*dst);
    int sizes[4] = {type_size(dst->typenum), 1, 1, 1};
    EwPlan plan;
    DPB_TRY(make_ew_plan(1, dst->nd, dst->shape, st.data(), sizes, plan));
    void *pout = const_cast<char *>(byte_ptr(dst->data, plan.offsets[0], dst->typenum));
    const void *pin[3] = {nullptr, nullptr, nullptr};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define DPB_FILL_CASE(B)                          \
    case B: {                                     \
        FillF<B> f;                               \
        std::memcpy(&f.v, scalar_bits, B);       \
        return launch_ew(f, plan, pin, pout, s);  \
    }
    switch (type_size(dst->typenum)) {
        DPB_FILL_CASE(1)
        DPB_FILL_CASE(2)
        DPB_FILL_CASE(4)
        DPB_FILL_CASE(8)
        DPB_FILL_CASE(16)
    }
#undef DPB_FILL_CASE
    return set_error(DPB_ERR_RUNTIME, "unsupported element size");
}

}  // extern "C"
