// Typed launcher of the reduction engine: turns a RedPlan into one or two
// kernel launches for a reduction operator R.
#pragma once

#include <algorithm>

#include "reduce_kernels.cuh"
#include "reduce_plan.h"

namespace dpb {

inline RedMeta make_meta(int nd, const int64_t *shape, const int64_t *s0, const int64_t *s1)
{
    RedMeta m;
    m.nd = nd;
    m.use64 = 0;
    for (int i = 0; i < kMaxD; ++i) {
        m.shape[i] = 1;
        m.strides[0][i] = 0;
        m.strides[1][i] = 0;
        m.div[i] = FastDiv32(1);
    }
    for (int i = 0; i < nd; ++i) {
        m.shape[i] = shape[i];
        m.strides[0][i] = s0 ? s0[i] : 0;
        m.strides[1][i] = s1 ? s1[i] : 0;
        if (shape[i] >= (int64_t(1) << 31)) m.use64 = 1;
        else m.div[i] = FastDiv32(static_cast<uint32_t>(shape[i] > 0 ? shape[i] : 1));
    }
    return m;
}

// dense C-order strides of `shape`, scaled by `scale`
inline void dense_strides(int nd, const int64_t *shape, int64_t scale, int64_t *out)
{
    int64_t acc = scale;
    for (int i = nd - 1; i >= 0; --i) {
        out[i] = acc;
        acc *= shape[i];
    }
}

inline int red_grid(int64_t nblocks)
{
    const int64_t cap = int64_t(device_props().sm_count) * tuning_ctas_per_sm();
    return static_cast<int>(std::max<int64_t>(1, std::min(nblocks, cap)));
}

inline int64_t red_target_blocks()
{
    return int64_t(device_props().sm_count) * tuning_ctas_per_sm();
}

template <class R> constexpr int inner_vec()
{
    constexpr int by_load = 16 / static_cast<int>(sizeof(typename R::In));
    constexpr int by_acc = 128 / static_cast<int>(sizeof(typename R::Acc));
    constexpr int v = by_load < by_acc ? by_load : by_acc;
    return v < 1 ? 1 : v;
}

template <class R> constexpr int outer_vec()
{
    constexpr int by_load = 16 / static_cast<int>(sizeof(typename R::In));
    constexpr int by_acc = 64 / static_cast<int>(sizeof(typename R::Acc));
    int v = by_load < by_acc ? by_load : by_acc;
    if (v > 4) v = 4;
    return v < 1 ? 1 : v;
}

// Writes the finished identity to every result (reduction over zero elements).
template <class R>
__global__ void reduce_identity_kernel(typename R::Out *res, RedMeta iter, int64_t niter)
{
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < niter;
         i += int64_t(gridDim.x) * blockDim.x) {
        int64_t o_src, o_dst;
        red_offsets(iter, i, o_src, o_dst);
        res[o_dst] = R::finish(R::identity());
    }
}

// ------------------------------------------------------------------ inner
// `final_pass` false: `res` is a dense scratch of Acc indexed [row][split].
template <class R>
int launch_inner(const typename R::In *arg, void *res, const RedMeta &iter, int64_t nrows, int64_t L,
                 int64_t nsplit, int64_t chunk, bool final_pass, cudaStream_t stream, int64_t index_rows = 1)
{
    constexpr int VEC = inner_vec<R>();
    constexpr int UNROLL = 4;
    const int64_t nitems = nrows * nsplit;
    const int64_t len = nsplit > 1 ? chunk : L;
    if (len <= 16) {
        launch_after_previous(reduce_inner_kernel<R, 1, 1, UNROLL>, red_grid(ceil_div(nitems, kRedThreads)), kRedThreads,
                              stream, arg, res, iter, nrows, L, nsplit, chunk, final_pass, index_rows);
        note_kernel("reduce_inner_thread");
    }
    else if (len <= 1024) {
        launch_after_previous(reduce_inner_kernel<R, VEC, 32, UNROLL>, red_grid(ceil_div(nitems, kRedThreads / 32)),
                              kRedThreads, stream, arg, res, iter, nrows, L, nsplit, chunk, final_pass, index_rows);
        note_kernel("reduce_inner_warp");
    }
    else {
        launch_after_previous(reduce_inner_kernel<R, VEC, 256, UNROLL>, red_grid(nitems), kRedThreads, stream, arg, res,
                              iter, nrows, L, nsplit, chunk, final_pass, index_rows);
        note_kernel("reduce_inner_block");
    }
    return check_launch("reduce_inner");
}

// Complete inner reduction including the split decision and the second pass.  The last
// reduction dimension is unit-stride; any further reduction dimensions ("outer" ones) are
// treated like extra rows whose partial results are merged by the second pass, in order.
template <class R>
int run_inner(const RedPlan &plan, const typename R::In *arg, void *res, cudaStream_t stream)
{
    using Acc = typename R::Acc;
    const int rlast = plan.red_nd - 1;
    const int64_t L = plan.red_nd > 0 ? plan.red_shape[rlast] : 1;
    int64_t n_outer = 1;
    for (int i = 0; i < rlast; ++i) n_outer *= plan.red_shape[i];
    const int64_t nrows = plan.niter * n_outer;
    // rows = iteration dimensions followed by the outer reduction dimensions
    int64_t shape[kMaxD], src[kMaxD], dst[kMaxD];
    int nd = 0;
    for (int i = 0; i < plan.iter_nd; ++i, ++nd) {
        shape[nd] = plan.iter_shape[i];
        src[nd] = plan.iter_src[i];
        dst[nd] = plan.iter_dst[i];
    }
    for (int i = 0; i < rlast; ++i, ++nd) {
        shape[nd] = plan.red_shape[i];
        src[nd] = plan.red_src[i];
        dst[nd] = 0;
    }
    RedMeta iter = make_meta(nd, shape, src, dst);
    int64_t nsplit = 1, chunk = L;
    const int64_t target = red_target_blocks();
    if (L > 16384 && nrows < target) {
        nsplit = std::min<int64_t>(ceil_div(target, nrows), L / 8192);
        nsplit = std::max<int64_t>(1, std::min<int64_t>(nsplit, 2048));
        chunk = ceil_div(ceil_div(L, nsplit), 1024) * 1024;
        nsplit = ceil_div(L, chunk);
    }
    if (nsplit <= 1 && n_outer == 1) return launch_inner<R>(arg, res, iter, nrows, L, 1, L, true, stream);

    void *scratch = nullptr;
    DPB_TRY(dpb_malloc(static_cast<size_t>(nrows * nsplit) * sizeof(Acc), stream, &scratch));
    int st = launch_inner<R>(arg, scratch, iter, nrows, L, nsplit, chunk, false, stream, n_outer);
    if (st == DPB_OK) {
        // partials are laid out [result][outer row][split]: one dense row per result
        const int64_t L2 = n_outer * nsplit;
        int64_t s2[kMaxD];
        dense_strides(plan.iter_nd, plan.iter_shape, L2, s2);
        RedMeta iter2 = make_meta(plan.iter_nd, plan.iter_shape, s2, plan.iter_dst);
        st = launch_inner<typename R::Stage2>(static_cast<const Acc *>(scratch), res, iter2, plan.niter, L2, 1,
                                              L2, true, stream);
    }
    dpb_free(scratch, stream);
    return st;
}

// ------------------------------------------------------------------ outer
// `columns_per_thread`: every thread owns its columns over the whole reduction range (many
// columns, short range); otherwise 8 thread rows share the range of a 32-thread column group.
template <class R>
int launch_outer(const typename R::In *arg, void *res, const RedMeta &batch, const RedMeta &red,
                 int64_t C, int64_t nred, int64_t nbatch, int64_t nslab, int64_t slab_len,
                 bool vector_ok, bool final_pass, cudaStream_t stream, bool columns_per_thread = false)
{
    constexpr int VEC = outer_vec<R>();
    constexpr int UNROLL = 4;
    const bool vec = vector_ok && VEC > 1;
    // the searches count rows inside a slab in 32 bits
    if (slab_len > 0x7fffffff) return set_error(DPB_ERR_RUNTIME, "reduction range of %lld rows is too long", static_cast<long long>(slab_len));
    if (columns_per_thread) {
        const int64_t ncg = ceil_div(C, int64_t(kRedThreads) * (vec ? VEC : 1));
        const int64_t nblocks = nbatch * nslab * ncg;
        const int grid = static_cast<int>(std::min<int64_t>(nblocks, int64_t(1) << 30));
        // loads in flight per thread: fewer for wide accumulators (value + index), which
        // otherwise cost the registers that occupancy needs
        constexpr int UC = (sizeof(typename R::Acc) > 8 && !R::kVectorStep) ? UNROLL : 2 * UNROLL;
        if (vec)
            launch_after_previous(reduce_outer_kernel<R, VEC, UC, 1>, grid, kRedThreads, stream, arg, res, batch, red, C,
                                  nred, nbatch, nslab, slab_len, ncg, final_pass);
        else
            launch_after_previous(reduce_outer_kernel<R, 1, UC, 1>, grid, kRedThreads, stream, arg, res, batch, red, C,
                                  nred, nbatch, nslab, slab_len, ncg, final_pass);
        note_kernel(vec ? "reduce_outer_cols_vec" : "reduce_outer_cols_scalar");
    }
    else if (vec) {
        const int64_t ncg = ceil_div(C, 32 * VEC);
        launch_after_previous(reduce_outer_kernel<R, VEC, UNROLL, kOuterRows>, red_grid(nbatch * nslab * ncg),
                              kRedThreads, stream, arg, res, batch, red, C, nred, nbatch, nslab, slab_len, ncg,
                              final_pass);
        note_kernel("reduce_outer_vec");
    }
    else {
        const int64_t ncg = ceil_div(C, 32);
        launch_after_previous(reduce_outer_kernel<R, 1, UNROLL, kOuterRows>, red_grid(nbatch * nslab * ncg),
                              kRedThreads, stream, arg, res, batch, red, C, nred, nbatch, nslab, slab_len, ncg,
                              final_pass);
        note_kernel("reduce_outer_scalar");
    }
    return check_launch("reduce_outer");
}

template <class R>
int run_outer(const RedPlan &plan, const typename R::In *arg, void *res, cudaStream_t stream)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    constexpr int VEC = outer_vec<R>();
    const int last = plan.iter_nd - 1;
    const int64_t C = plan.iter_shape[last];
    const int64_t nbatch = plan.niter / C;
    const int64_t nred = plan.nred;
    RedMeta batch = make_meta(last, plan.iter_shape, plan.iter_src, plan.iter_dst);
    RedMeta red = make_meta(plan.red_nd, plan.red_shape, plan.red_src, nullptr);

    bool vector_ok = (C % VEC == 0) && is_aligned(arg, sizeof(In) * VEC);
    for (int i = 0; i < last; ++i) vector_ok = vector_ok && (plan.iter_src[i] % VEC == 0);
    for (int i = 0; i < plan.red_nd; ++i) vector_ok = vector_ok && (plan.red_src[i] % VEC == 0);
    const int vec = (vector_ok && VEC > 1) ? VEC : 1;

    const int64_t target = red_target_blocks();
    // enough columns to give every thread its own: no sharing of the reduction range
    if (nbatch * ceil_div(C, int64_t(kRedThreads) * vec) >= 4 * int64_t(device_props().sm_count))
        return launch_outer<R>(arg, res, batch, red, C, nred, nbatch, 1, nred, vector_ok, true, stream, true);

    const int64_t work0 = nbatch * ceil_div(C, 32 * vec);
    int64_t nslab = 1, slab_len = nred;
    if (work0 * 2 <= target && nred >= 128) {
        nslab = std::min<int64_t>(ceil_div(target, work0), nred / 64);
        nslab = std::max<int64_t>(1, std::min<int64_t>(nslab, 1024));
        slab_len = ceil_div(ceil_div(nred, nslab), 32) * 32;
        nslab = ceil_div(nred, slab_len);
    }
    if (nslab <= 1)
        return launch_outer<R>(arg, res, batch, red, C, nred, nbatch, 1, nred, vector_ok, true, stream);

    void *scratch = nullptr;
    DPB_TRY(dpb_malloc(static_cast<size_t>(nslab * nbatch * C) * sizeof(Acc), stream, &scratch));
    int st = launch_outer<R>(arg, scratch, batch, red, C, nred, nbatch, nslab, slab_len, vector_ok,
                             false, stream);
    if (st == DPB_OK) {
        using R2 = typename R::Stage2;
        constexpr int VEC2 = outer_vec<R2>();
        int64_t s2[kMaxD];
        dense_strides(last, plan.iter_shape, C, s2);
        RedMeta batch2 = make_meta(last, plan.iter_shape, s2, plan.iter_dst);
        const int64_t rs = nbatch * C;
        RedMeta red2 = make_meta(1, &nslab, &rs, nullptr);
        st = launch_outer<R2>(static_cast<const Acc *>(scratch), res, batch2, red2, C, nslab, nbatch, 1,
                              nslab, C % VEC2 == 0, true, stream);
    }
    dpb_free(scratch, stream);
    return st;
}

// ---------------------------------------------------------------- generic
template <class R>
int run_generic(const RedPlan &plan, const typename R::In *arg, void *res, cudaStream_t stream)
{
    using Acc = typename R::Acc;
    RedMeta iter = make_meta(plan.iter_nd, plan.iter_shape, plan.iter_src, plan.iter_dst);
    RedMeta red = make_meta(plan.red_nd, plan.red_shape, plan.red_src, nullptr);
    const int64_t niter = plan.niter, nred = plan.nred;
    const int64_t target = red_target_blocks();
    if (nred <= 1024 || niter >= target * 8) {
        reduce_generic_kernel<R, 32><<<red_grid(ceil_div(niter, kRedThreads / 32)), kRedThreads, 0,
                                       stream>>>(arg, res, iter, red, niter, nred, 1, nred, true);
        note_kernel("reduce_generic_warp");
        return check_launch("reduce_generic");
    }
    int64_t nsplit = 1, chunk = nred;
    if (niter < target && nred > 16384) {
        nsplit = std::min<int64_t>(ceil_div(target, niter), nred / 4096);
        nsplit = std::max<int64_t>(1, std::min<int64_t>(nsplit, 2048));
        chunk = ceil_div(nred, nsplit);
        nsplit = ceil_div(nred, chunk);
    }
    if (nsplit <= 1) {
        reduce_generic_kernel<R, 256>
            <<<red_grid(niter), kRedThreads, 0, stream>>>(arg, res, iter, red, niter, nred, 1, nred, true);
        note_kernel("reduce_generic_block");
        return check_launch("reduce_generic");
    }
    void *scratch = nullptr;
    DPB_TRY(dpb_malloc(static_cast<size_t>(niter * nsplit) * sizeof(Acc), stream, &scratch));
    reduce_generic_kernel<R, 256><<<red_grid(niter * nsplit), kRedThreads, 0, stream>>>(
        arg, scratch, iter, red, niter, nred, nsplit, chunk, false);
    note_kernel("reduce_generic_block");
    int st = check_launch("reduce_generic");
    if (st == DPB_OK) {
        int64_t s2[kMaxD];
        dense_strides(plan.iter_nd, plan.iter_shape, nsplit, s2);
        RedMeta iter2 = make_meta(plan.iter_nd, plan.iter_shape, s2, plan.iter_dst);
        st = launch_inner<typename R::Stage2>(static_cast<const Acc *>(scratch), res, iter2, niter,
                                              nsplit, 1, nsplit, true, stream);
    }
    dpb_free(scratch, stream);
    return st;
}

// Entry: `arg` and `res` are already displaced by the plan's offsets.
template <class R>
int launch_reduction(const RedPlan &plan, const void *arg, void *res, cudaStream_t stream)
{
    using In = typename R::In;
    if (plan.niter == 0) return DPB_OK;
    if (plan.nred == 0) {
        RedMeta iter = make_meta(plan.iter_nd, plan.iter_shape, plan.iter_src, plan.iter_dst);
        reduce_identity_kernel<R><<<red_grid(ceil_div(plan.niter, 256)), 256, 0, stream>>>(
            static_cast<typename R::Out *>(res), iter, plan.niter);
        note_kernel("reduce_identity");
        return check_launch("reduce_identity");
    }
    const In *a = static_cast<const In *>(arg);
    switch (plan.kind) {
    case RED_INNER: return run_inner<R>(plan, a, res, stream);
    case RED_OUTER: return run_outer<R>(plan, a, res, stream);
    default: return run_generic<R>(plan, a, res, stream);
    }
}

}  // namespace dpb
