// Accumulation over the last axis: tables, launch plan and the C entry point
// dpb_accumulate_over_axis.  Argument checks follow py_accumulate_over_axis /
// py_accumulate_final_axis_include_initial
// (dpnp/tensor/libtensor/source/accumulators/accumulate_over_axis.hpp:74-260,262-460).
#include <mutex>
#include <vector>

#include "iterspace.h"
#include "reduce_register.cuh"
#include "scan_kernels.cuh"

#ifndef DPB_SCAN_MIN_ITEMS
#define DPB_SCAN_MIN_ITEMS 8
#endif

namespace dpb {

// probes per wait of the single-pass scan; -1: long rows take the three-launch path instead
int64_t tuning_scan_lookback_polls();

struct ScanPlan {
    RedMeta iter;        // leading (not scanned) dimensions, collapsed; strides of src and dst
    int iter_nd = 0;
    int64_t iter_shape[kMaxD], iter_src[kMaxD], iter_dst[kMaxD];
    int64_t nrows = 1;
    int64_t L = 0, s_src = 1, s_dst = 1;
    int64_t dst_shift = 0;
};

typedef int (*scan_fn_t)(const ScanPlan &plan, const void *src, void *dst, cudaStream_t stream);

// Elements per thread and chunk: 8 for types of 4 bytes and more (two 16-byte loads of float32 in
// flight per thread; measured on B200, cumsum of 16384 x 65536 float32 along the rows: 8 elements
// 1.32 ms, 16 elements 1.53 ms -- the smaller chunk needs half the registers, so twice the
// blocks are resident and a row's chunks follow each other faster), up to 16 for narrower types,
// bounded by the registers the accumulators take.
template <class R> constexpr int scan_items()
{
    constexpr int by_in = 32 / static_cast<int>(sizeof(typename R::In));
    constexpr int by_acc = 128 / static_cast<int>(sizeof(typename R::Acc));
    constexpr int v = by_in < by_acc ? by_in : by_acc;
    return v < DPB_SCAN_MIN_ITEMS ? DPB_SCAN_MIN_ITEMS : (v > 16 ? 16 : v);
}

// The single-pass scan pays one round of probes per tile: larger tiles (four 16-byte loads of
// float32 per thread) were measured faster there (0.94 ms against 1.54 ms with 8 elements).
template <class R> constexpr int lookback_items()
{
    constexpr int by_in = 64 / static_cast<int>(sizeof(typename R::In));
    constexpr int by_acc = 128 / static_cast<int>(sizeof(typename R::Acc));
    constexpr int v = by_in < by_acc ? by_in : by_acc;
    return v < 2 ? 2 : (v > 16 ? 16 : v);
}

template <class R>
__global__ void scan_fill_identity_kernel(typename R::Out *dst, RedMeta iter, int64_t nrows)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nrows; i += int64_t(gridDim.x) * blockDim.x) {
        int64_t o_src, o_dst;
        red_offsets(iter, i, o_src, o_dst);
        dst[o_dst] = R::finish(R::identity());
    }
}

template <class R> int launch_scan(const ScanPlan &plan, const void *vsrc, void *vdst, cudaStream_t stream)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    using Out = typename R::Out;
    constexpr int ITEMS = scan_items<R>();
    const In *src = static_cast<const In *>(vsrc);
    Out *dst = static_cast<Out *>(vdst);
    const int64_t nrows = plan.nrows, L = plan.L;
    if (plan.dst_shift) {
        // position 0 of every row holds the identity (accumulate_over_axis.hpp:262-460)
        scan_fill_identity_kernel<R><<<red_grid(ceil_div(nrows, 256)), 256, 0, stream>>>(dst, plan.iter, nrows);
        note_kernel("scan_fill_identity");
        DPB_TRY(check_launch("scan_fill_identity"));
    }
    if (L == 0) return DPB_OK;
    const int64_t target = red_target_blocks();

    // columns: the innermost leading dimension is unit-stride on both sides and long enough
    const int last = plan.iter_nd - 1;
    if (plan.iter_nd >= 1 && plan.iter_src[last] == 1 && plan.iter_dst[last] == 1 &&
        (plan.s_src != 1 || plan.s_dst != 1)) {
        const int64_t cols = plan.iter_shape[last];
        const int64_t nbatch = nrows / cols;
        if (cols >= 32 && nbatch * ceil_div(cols, 256) >= int64_t(device_props().sm_count)) {
            RedMeta batch = make_meta(last, plan.iter_shape, plan.iter_src, plan.iter_dst);
            const int64_t nwork = nbatch * ceil_div(cols, kScanColThreads);
            scan_cols_kernel<R><<<static_cast<int>(std::min<int64_t>(nwork, int64_t(1) << 30)), kScanColThreads, 0,
                                  stream>>>(src, dst, batch, nbatch, cols, L, plan.s_src, plan.s_dst,
                                            plan.dst_shift);
            note_kernel("scan_cols");
            return check_launch("scan_cols");
        }
    }

    const bool unit = plan.s_src == 1 && plan.s_dst == 1;
    // whole-thread vector accesses: rows start on the vector grid in both arrays
    // (a thread's first element is a multiple of ITEMS, and ITEMS elements are whole 16-byte
    // pieces of either type, so 16-byte aligned row starts are all that is needed)
    constexpr int64_t in16 = sizeof(In) >= 16 ? 1 : 16 / sizeof(In);
    constexpr int64_t out16 = sizeof(Out) >= 16 ? 1 : 16 / sizeof(Out);
    bool vec = unit && plan.dst_shift == 0 && ITEMS % in16 == 0 && ITEMS % out16 == 0 &&
               is_aligned(src, 16) && is_aligned(dst, 16);
    for (int i = 0; i < plan.iter_nd; ++i)
        vec = vec && plan.iter_src[i] % in16 == 0 && plan.iter_dst[i] % out16 == 0;
    const int64_t chunk = int64_t(kScanThreads) * ITEMS;
    int64_t nseg = 1, seg_len = L;
    if (nrows < target && L > 4 * chunk) {
        nseg = std::min<int64_t>(ceil_div(target, nrows), L / (2 * chunk));
        nseg = std::max<int64_t>(1, std::min<int64_t>(nseg, 4096));
        seg_len = ceil_div(ceil_div(L, nseg), chunk) * chunk;
        nseg = ceil_div(L, seg_len);
    }
    // A few long unit-stride rows: one pass over the data, tiles chained through published totals
    // (scan_lookback_kernel).  The two repair launches return at once unless a wait ran out.
    const int64_t polls = tuning_scan_lookback_polls();
    constexpr int LB_ITEMS = lookback_items<R>();
    const int64_t ntiles = ceil_div(L, int64_t(kScanThreads) * LB_ITEMS);
    const bool lb_vec = vec && LB_ITEMS % in16 == 0 && LB_ITEMS % out16 == 0;
    if (nseg > 1 && unit && polls >= 0 && nrows * ntiles < (int64_t(1) << 30)) {
        LookbackLayout lay;
        lay.levels = 0;
        lay.per_row = 0;
        for (int64_t cnt = ntiles; lay.levels < kLookbackLevels; cnt = ceil_div(cnt, 32)) {
            lay.n[lay.levels] = cnt;
            lay.off[lay.levels] = lay.per_row;
            lay.per_row += cnt;
            ++lay.levels;
            if (cnt <= 32) break;
        }
        for (int i = lay.levels; i < kLookbackLevels; ++i) lay.n[i] = lay.off[i] = 0;
        if (lay.n[lay.levels - 1] <= 32) {
            const int64_t entries = nrows * lay.per_row, tiles = nrows * ntiles;
            // values | flags | done words | error
            using Entries = LookbackEntries<Acc>;
            const size_t val_bytes = (static_cast<size_t>(entries) * Entries::kValueBytes + 15) / 16 * 16;
            const size_t word_bytes = static_cast<size_t>(entries + tiles + 1) * sizeof(unsigned);
            void *scratch = nullptr;
            DPB_TRY(dpb_malloc(val_bytes + word_bytes, stream, &scratch));
            Entries ent;
            ent.vals = scratch;
            ent.flags = reinterpret_cast<unsigned *>(static_cast<char *>(scratch) + val_bytes);
            unsigned *done = ent.flags + entries, *error = done + tiles;
            int st = DPB_OK;
            if (cudaMemsetAsync(scratch, 0, val_bytes + word_bytes, stream) != cudaSuccess) {
                cudaGetLastError();
                st = set_error(DPB_ERR_CUDA, "scan: clearing the entries failed");
            }
            note_copy("memset");
            const int max_polls = static_cast<int>(std::min<int64_t>(polls, int64_t(1) << 30));
#define DPB_LOOKBACK_LAUNCH(VEC)                                                                      \
    scan_lookback_kernel<R, LB_ITEMS, VEC><<<static_cast<int>(tiles), kScanThreads, 0, stream>>>(          \
        src, dst, plan.iter, L, ntiles, lay, ent, done, error, max_polls, plan.dst_shift)
#define DPB_LOOKBACK_REPAIR(VEC)                                                                      \
    scan_lookback_repair_kernel<R, LB_ITEMS, VEC><<<red_grid(tiles), kScanThreads, 0, stream>>>(           \
        src, dst, plan.iter, nrows, L, ntiles, lay, ent, done, error, plan.dst_shift)
            if (st == DPB_OK) {
                if (lb_vec) DPB_LOOKBACK_LAUNCH(true);
                else DPB_LOOKBACK_LAUNCH(false);
                st = check_launch("scan_lookback");
            }
            if (st == DPB_OK) {
                scan_lookback_levels_kernel<R><<<1, 1024, 0, stream>>>(ent, lay, nrows, error);
                note_kernel("scan_lookback_levels");
                st = check_launch("scan_lookback_levels");
            }
            if (st == DPB_OK) {
                if (lb_vec) DPB_LOOKBACK_REPAIR(true);
                else DPB_LOOKBACK_REPAIR(false);
                note_kernel("scan_lookback_repair");
                st = check_launch("scan_lookback_repair");
            }
            note_kernel(lb_vec ? "scan_lookback_vec" : "scan_lookback");   // the pass that does the work, named last
#undef DPB_LOOKBACK_REPAIR
#undef DPB_LOOKBACK_LAUNCH
            dpb_free(scratch, stream);
            return st;
        }
    }
    const int grid = red_grid(nrows * nseg);
#define DPB_SCAN_LAUNCH(UNIT, VEC, TOT, CARRY, TOTALS)                                                  \
    scan_rows_kernel<R, ITEMS, UNIT, VEC, TOT><<<grid, kScanThreads, 0, stream>>>(                      \
        src, dst, plan.iter, nrows, L, plan.s_src, plan.s_dst, nseg, seg_len, CARRY, TOTALS, plan.dst_shift)
    Acc *totals = nullptr;
    if (nseg > 1) {
        void *scratch = nullptr;
        DPB_TRY(dpb_malloc(static_cast<size_t>(nrows * nseg) * sizeof(Acc), stream, &scratch));
        totals = static_cast<Acc *>(scratch);
        if (vec) DPB_SCAN_LAUNCH(true, true, true, nullptr, totals);
        else if (unit) DPB_SCAN_LAUNCH(true, false, true, nullptr, totals);
        else DPB_SCAN_LAUNCH(false, false, true, nullptr, totals);
        note_kernel("scan_rows_totals");
        int st = check_launch("scan_rows_totals");
        if (st == DPB_OK) {
            scan_totals_kernel<R><<<static_cast<int>(ceil_div(nrows, kScanThreads / 32)), kScanThreads, 0, stream>>>(
                totals, nrows, nseg);
            note_kernel("scan_totals");
            st = check_launch("scan_totals");
        }
        if (st != DPB_OK) {
            dpb_free(scratch, stream);
            return st;
        }
    }
    if (vec) DPB_SCAN_LAUNCH(true, true, false, totals, nullptr);
    else if (unit) DPB_SCAN_LAUNCH(true, false, false, totals, nullptr);
    else DPB_SCAN_LAUNCH(false, false, false, totals, nullptr);
#undef DPB_SCAN_LAUNCH
    note_kernel(vec ? "scan_rows_vec" : (unit ? "scan_rows" : "scan_rows_strided"));
    const int st = check_launch("scan_rows");
    if (totals) dpb_free(totals, stream);
    return st;
}

template <class R> int scan_entry(const ScanPlan &plan, const void *src, void *dst, cudaStream_t stream)
{
    return launch_scan<R>(plan, src, dst, stream);
}

struct ScanTables {
    scan_fn_t fn[DPB_A_NUM_OPS][DPB_NUM_TYPES][DPB_NUM_TYPES];
};

template <template <class, class> class Red, bool FP_ONLY, int TI, int TO> void reg_scan_one(scan_fn_t (*tab)[DPB_NUM_TYPES])
{
    using I = type_of_t<TI>;
    using O = type_of_t<TO>;
    if constexpr (FP_ONLY ? fp_pair_v<I, O> : accumulate_pair_v<I, O>)
        tab[TI][TO] = &scan_entry<Red<I, O>>;
}
template <template <class, class> class Red, bool FP_ONLY, int TI, int... TO>
void reg_scan_row(scan_fn_t (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TO...>)
{
    (reg_scan_one<Red, FP_ONLY, TI, TO>(tab), ...);
}
template <template <class, class> class Red, bool FP_ONLY, int... TI>
void reg_scan(scan_fn_t (*tab)[DPB_NUM_TYPES], std::integer_sequence<int, TI...>)
{
    (reg_scan_row<Red, FP_ONLY, TI>(tab, std::make_integer_sequence<int, DPB_NUM_TYPES>()), ...);
}

template <class I, class O> using CumSumPair = SumRed<I, O>;
template <class I, class O> using CumProdPair = ProdRed<I, O>;
template <class I, class O> using CumLogSumExpPair = LogSumExpRed<I, O>;

static ScanTables g_scan;
static std::once_flag g_scan_once;

static const ScanTables &scan_tables()
{
    std::call_once(g_scan_once, [] {
        constexpr auto all = std::make_integer_sequence<int, DPB_NUM_TYPES>();
        reg_scan<CumSumPair, false>(g_scan.fn[DPB_A_CUMSUM], all);
        reg_scan<CumProdPair, false>(g_scan.fn[DPB_A_CUMPROD], all);
        reg_scan<CumLogSumExpPair, true>(g_scan.fn[DPB_A_CUMLOGSUMEXP], all);
    });
    return g_scan;
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_accumulate_dtype_supported(int op, int t_in, int t_out)
{
    if (op < 0 || op >= DPB_A_NUM_OPS || t_in < 0 || t_in >= DPB_NUM_TYPES || t_out < 0 || t_out >= DPB_NUM_TYPES)
        return 0;
    return scan_tables().fn[op][t_in][t_out] != nullptr;
}

extern "C" int dpb_accumulate_over_axis(int op, const dpb_array *src, const dpb_array *dst, int include_initial,
                                        void *stream)
{
    DPB_TRY(check_array(src, "src"));
    DPB_TRY(check_array(dst, "dst"));
    if (op < 0 || op >= DPB_A_NUM_OPS) return set_error(DPB_ERR_VALUE, "unknown accumulation op %d", op);
    if (src->nd < 1) return set_error(DPB_ERR_VALUE, "The input array must have at least one dimension");
    if (src->nd != dst->nd) return set_error(DPB_ERR_VALUE, "The input and output arrays must have the same array ranks");
    const int nd = src->nd, lead = nd - 1;
    for (int i = 0; i < lead; ++i)
        if (src->shape[i] != dst->shape[i])
            return set_error(DPB_ERR_VALUE, "Destination shape does not match the input shape");
    const int64_t L = src->shape[lead];
    if (dst->shape[lead] != L + (include_initial ? 1 : 0))
        return set_error(DPB_ERR_VALUE, "Destination shape does not match the input shape");
    if (src->device != dst->device)
        return set_error(DPB_ERR_VALUE, "Execution queue is not compatible with allocation queues");
    if (!(dst->flags & DPB_FLAG_WRITABLE)) return set_error(DPB_ERR_VALUE, "output array is read-only.");
    if (num_elements(*dst) == 0) return DPB_OK;
    if (arrays_overlap(*src, *dst) && !same_logical_tensors(*src, *dst))
        return set_error(DPB_ERR_VALUE, "Arrays index overlapping segments of memory");
    const scan_fn_t fn = scan_tables().fn[op][src->typenum][dst->typenum];
    if (!fn) return set_error(DPB_ERR_RUNTIME, "Datatypes are not supported");

    std::vector<int64_t> ss = strides_of(*src), ds = strides_of(*dst);
    ScanPlan plan;
    plan.L = L;
    plan.s_src = ss[lead];
    plan.s_dst = ds[lead];
    plan.dst_shift = include_initial ? 1 : 0;
    // collapse the leading dimensions of both arrays together
    std::vector<int64_t> shape(src->shape, src->shape + lead), strides(2 * size_t(lead > 0 ? lead : 1));
    for (int i = 0; i < lead; ++i) {
        strides[i] = ss[i];
        strides[lead + i] = ds[i];
    }
    int64_t offsets[kMaxArrays] = {0, 0, 0, 0};
    int cnd = lead > 0 ? simplify_iteration_space(2, lead, shape.data(), strides.data(), offsets) : 0;
    if (cnd > kMaxD) return set_error(DPB_ERR_RUNTIME, "too many dimensions remain after collapsing");
    plan.iter_nd = cnd;
    plan.nrows = 1;
    for (int i = 0; i < cnd; ++i) {
        plan.iter_shape[i] = shape[i];
        plan.iter_src[i] = strides[i];
        plan.iter_dst[i] = strides[cnd + i];   // collapsed strides are repacked [array][cnd]
        plan.nrows *= shape[i];
    }
    plan.iter = make_meta(cnd, plan.iter_shape, plan.iter_src, plan.iter_dst);
    const char *a = static_cast<const char *>(src->data) + offsets[0] * type_size(src->typenum);
    char *r = static_cast<char *>(dst->data) + offsets[1] * type_size(dst->typenum);
    return fn(plan, a, r, static_cast<cudaStream_t>(stream));
}
