// Reduction engine: kernel templates for any reduction operator R (see
// reduce_ops.cuh).  Three kernel shapes cover every layout:
//   reduce_inner    the reduced elements of one result are contiguous in
//                   memory ("rows"); GROUP threads (1, 32 or 256) cooperate on a
//                   row, long rows are split over several blocks
//   reduce_outer    the results are contiguous in memory ("columns") and the
//                   reduction walks rows: each thread owns VEC adjacent columns
//                   so every access is coalesced; rows are split into slabs
//   reduce_generic  arbitrary strides on both sides, offsets from collapsed
//                   shape/strides held in kernel parameters
// Work is partitioned by the sizes alone and combined in a fixed order, so the
// result of a floating-point sum does not change from run to run.  When a
// reduction is split, partial accumulators go to a scratch buffer and a second
// launch of the same kernels (with R::Stage2) merges them.
//
// These replace the reference kernels of include/kernels/reductions.hpp:
// SequentialReduction (:98-152), ReductionOverGroupWithAtomicFunctor (:161-287),
// ReductionOverGroupNoAtomicFunctor (:419-517), SearchReduction (:1988-2131) and
// their axis1/axis0/strided launchers (:757-1046,1137-1856,2487-3308).
#pragma once

#include <cstring>

#include "common.cuh"
#include "ew_plan.h"
#include "reduce_ops.cuh"

namespace dpb {

constexpr int kRedThreads = 256;

// Collapsed dimensions of one side of a reduction: `nd` extents with the
// strides of up to two arrays, plus multiply-shift dividers.
struct RedMeta {
    int nd;
    int use64;  // an extent does not fit 31 bits: use 64-bit division
    int64_t shape[kMaxD];
    int64_t strides[2][kMaxD];
    FastDiv32 div[kMaxD];
};

// linear index (C order over m.shape) -> element offsets in both arrays
DPB_D void red_offsets(const RedMeta &m, int64_t lin, int64_t &o0, int64_t &o1)
{
    o0 = 0;
    o1 = 0;
    if (m.nd == 0) return;
    if (!m.use64 && lin < (int64_t(1) << 31)) {
        uint32_t rem = static_cast<uint32_t>(lin);
        for (int d = m.nd - 1; d > 0; --d) {
            uint32_t q, r;
            m.div[d].divmod(rem, q, r);
            rem = q;
            o0 += int64_t(r) * m.strides[0][d];
            o1 += int64_t(r) * m.strides[1][d];
        }
        o0 += int64_t(rem) * m.strides[0][0];
        o1 += int64_t(rem) * m.strides[1][0];
    }
    else {
        int64_t rem = lin;
        for (int d = m.nd - 1; d > 0; --d) {
            const int64_t q = rem / m.shape[d];
            const int64_t r = rem - q * m.shape[d];
            rem = q;
            o0 += r * m.strides[0][d];
            o1 += r * m.strides[1][d];
        }
        o0 += rem * m.strides[0][0];
        o1 += rem * m.strides[1][0];
    }
}

// ---------------------------------------------------------------- shuffles
template <class T> DPB_D T shfl_down_any(const T &v, int delta)
{
    constexpr int W = (sizeof(T) + 3) / 4;
    uint32_t w[W];
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = 0;
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_down_sync(0xffffffffu, w[i], delta);
    T out;
    memcpy(&out, w, sizeof(T));
    return out;
}

template <class R> DPB_D typename R::Acc warp_reduce(typename R::Acc a)
{
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) a = R::combine(a, shfl_down_any(a, d));
    return a;  // valid in lane 0
}

// Reduce over a group of GROUP threads (1, 32 or 256); the result is valid in
// the first thread of the group.  `smem` needs 8 accumulators for GROUP 256.
template <class R, int GROUP> DPB_D typename R::Acc group_reduce(typename R::Acc a, typename R::Acc *smem)
{
    if constexpr (GROUP == 1) {
        return a;
    }
    else if constexpr (GROUP == 32) {
        return warp_reduce<R>(a);
    }
    else {
        a = warp_reduce<R>(a);
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        __syncthreads();  // protect smem from the previous use
        if (lane == 0) smem[warp] = a;
        __syncthreads();
        if (warp == 0) {
            typename R::Acc b = (lane < GROUP / 32) ? smem[lane] : R::identity();
            b = warp_reduce<R>(b);
            a = b;
        }
        return a;
    }
}

// Store either a partial accumulator (scratch, dense) or the finished result.
template <class R> DPB_D void red_store(void *res, int64_t index, const typename R::Acc &a, bool final_pass)
{
    if (final_pass) static_cast<typename R::Out *>(res)[index] = R::finish(a);
    else static_cast<typename R::Acc *>(res)[index] = a;
}

// ------------------------------------------------------------------- inner
// Work item = (row, split).  Row r starts at arg + offset(iter, r); split s
// covers reduction indices [s*chunk, min(L, (s+1)*chunk)).  The body is read
// with 16-byte loads after peeling elements up to the next 16-byte boundary.
template <class R, int VEC, int GROUP, int UNROLL>
__global__ void __launch_bounds__(kRedThreads)
    reduce_inner_kernel(const typename R::In *arg, void *res, RedMeta iter, int64_t nrows, int64_t L,
                        int64_t nsplit, int64_t chunk, bool final_pass, int64_t index_rows)
{
    cudaGridDependencySynchronize();   // see launch_after_previous
    using In = typename R::In;
    using Acc = typename R::Acc;
    __shared__ Acc smem[8];
    constexpr int GROUPS_PER_BLOCK = kRedThreads / GROUP;
    const int g = threadIdx.x / GROUP;   // group within the block
    const int t = threadIdx.x % GROUP;   // thread within the group
    const int64_t nitems = nrows * nsplit;
    const int64_t nblock_items = (nitems + GROUPS_PER_BLOCK - 1) / GROUPS_PER_BLOCK;

    for (int64_t bi = blockIdx.x; bi < nblock_items; bi += gridDim.x) {
        const int64_t item = bi * GROUPS_PER_BLOCK + g;
        const bool active = item < nitems;
        Acc acc = R::identity();
        int64_t row = 0, split = 0, o_src = 0, o_dst = 0;
        if (active) {
            row = item / nsplit;
            split = item - row * nsplit;
            red_offsets(iter, row, o_src, o_dst);
            const int64_t begin = split * chunk;
            int64_t len = L - begin;
            if (len > chunk) len = chunk;
            const In *p = arg + o_src + begin;
            // reduction index of the first element: rows that are slices of one result
            // (index_rows of them per result, in order) continue each other's numbering
            const int64_t ib = begin + (index_rows > 1 ? (row % index_rows) * L : 0);
            if constexpr (VEC > 1 && GROUP > 1) {
                // peel up to the next 16-byte boundary
                const uintptr_t addr = reinterpret_cast<uintptr_t>(p) / sizeof(In);
                int64_t head = static_cast<int64_t>((VEC - (addr % VEC)) % VEC);
                if (head > len) head = len;
                if (t < head) acc = R::step(acc, p[t], ib + t);
                const In *q = p + head;
                const int64_t nvec = (len - head) / VEC;
                if constexpr (R::kVectorStep) {
                    // one accumulator per load slot, fed a whole vector at a time
                    Acc la[UNROLL];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) la[u] = R::identity();
                    int64_t v = t;
                    for (; v + int64_t(UNROLL - 1) * GROUP < nvec; v += int64_t(UNROLL) * GROUP) {
                        vec_t<In, VEC> x[UNROLL];
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u)
                            x[u] = load_vec<vec_t<In, VEC>>(q + (v + int64_t(u) * GROUP) * VEC);
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u)
                            la[u] = R::template step_vec<VEC>(la[u], x[u].v,
                                                               ib + head + (v + int64_t(u) * GROUP) * VEC);
                    }
                    for (; v < nvec; v += GROUP) {
                        vec_t<In, VEC> x = load_vec<vec_t<In, VEC>>(q + v * VEC);
                        la[0] = R::template step_vec<VEC>(la[0], x.v, ib + head + v * VEC);
                    }
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) acc = R::combine(acc, la[u]);
                }
                else {
                    // independent accumulators per load slot only while they stay cheap
                    constexpr int LU = (sizeof(Acc) * VEC * UNROLL <= 256) ? UNROLL : 1;
                    Acc lanes[LU][VEC];
#pragma unroll
                    for (int u = 0; u < LU; ++u)
#pragma unroll
                        for (int k = 0; k < VEC; ++k) lanes[u][k] = R::identity();
                    int64_t v = t;
                    for (; v + int64_t(UNROLL - 1) * GROUP < nvec; v += int64_t(UNROLL) * GROUP) {
                        vec_t<In, VEC> x[UNROLL];
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u)
                            x[u] = load_vec<vec_t<In, VEC>>(q + (v + int64_t(u) * GROUP) * VEC);
#pragma unroll
                        for (int u = 0; u < UNROLL; ++u) {
                            const int64_t e0 = ib + head + (v + int64_t(u) * GROUP) * VEC;
#pragma unroll
                            for (int k = 0; k < VEC; ++k)
                                lanes[u % LU][k] = R::step(lanes[u % LU][k], x[u].v[k], e0 + k);
                        }
                    }
                    for (; v < nvec; v += GROUP) {
                        vec_t<In, VEC> x = load_vec<vec_t<In, VEC>>(q + v * VEC);
                        const int64_t e0 = ib + head + v * VEC;
#pragma unroll
                        for (int k = 0; k < VEC; ++k)
                            lanes[0][k] = R::step(lanes[0][k], x.v[k], e0 + k);
                    }
#pragma unroll
                    for (int u = 0; u < LU; ++u)
#pragma unroll
                        for (int k = 0; k < VEC; ++k) acc = R::combine(acc, lanes[u][k]);
                }
                const int64_t done = head + nvec * VEC;
                if (done + t < len) acc = R::step(acc, p[done + t], ib + done + t);
            }
            else {
                Acc lanes[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) lanes[u] = R::identity();
                int64_t e = t;
                for (; e + int64_t(UNROLL - 1) * GROUP < len; e += int64_t(UNROLL) * GROUP) {
                    In x[UNROLL];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) x[u] = p[e + int64_t(u) * GROUP];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u)
                        lanes[u] = R::step(lanes[u], x[u], ib + e + int64_t(u) * GROUP);
                }
                for (; e < len; e += GROUP) lanes[0] = R::step(lanes[0], p[e], ib + e);
#pragma unroll
                for (int u = 0; u < UNROLL; ++u) acc = R::combine(acc, lanes[u]);
            }
        }
        acc = group_reduce<R, GROUP>(acc, smem);
        if (active && t == 0) {
            if (final_pass) red_store<R>(res, o_dst, acc, true);
            else red_store<R>(res, item, acc, false);
        }
    }
}

// ------------------------------------------------------------------- outer
// Source seen as [batch][reduction rows][C columns], columns unit-stride in
// both source and result.  Block = 32 column-threads x 8 row-threads; thread
// (tx, ty) owns VEC adjacent columns and every 8th row of its slab.
// Work item = (batch entry, slab, column group); partials are stored densely
// as [slab][batch][C].
constexpr int kOuterRows = 8;

template <class R, int VEC, int UNROLL, int ROWS>
__global__ void __launch_bounds__(kRedThreads)
    reduce_outer_kernel(const typename R::In *arg, void *res, RedMeta batch, RedMeta red, int64_t C,
                        int64_t nred, int64_t nbatch, int64_t nslab, int64_t slab_len,
                        int64_t ncolgroups, bool final_pass)
{
    cudaGridDependencySynchronize();   // see launch_after_previous
    using In = typename R::In;
    using Acc = typename R::Acc;
    // ROWS thread rows share the reduction range of a column group; ROWS == 1 gives every
    // thread its own columns and needs no exchange through shared memory
    constexpr int TXW = kRedThreads / ROWS;
    __shared__ Acc smem[ROWS > 1 ? ROWS : 1][ROWS > 1 ? TXW : 1][VEC];
    const int tx = threadIdx.x % TXW, ty = threadIdx.x / TXW;
    const int64_t nwork = nbatch * nslab * ncolgroups;

    for (int64_t w = blockIdx.x; w < nwork; w += gridDim.x) {
        const int64_t cg = w % ncolgroups;
        const int64_t ws = w / ncolgroups;
        const int64_t slab = ws % nslab;
        const int64_t b = ws / nslab;
        const int64_t col = (cg * TXW + tx) * VEC;
        const bool active = col < C;
        int64_t b_src = 0, b_dst = 0;
        red_offsets(batch, b, b_src, b_dst);
        Acc lanes[VEC];
#pragma unroll
        for (int k = 0; k < VEC; ++k) lanes[k] = R::identity();
        if (active) {
            const In *base = arg + b_src + col;
            const int64_t r_begin = slab * slab_len;
            int64_t r_end = r_begin + slab_len;
            if (r_end > nred) r_end = nred;
            const bool simple = (red.nd == 1);
            const int64_t rs = red.strides[0][0];
            int64_t r = r_begin + ty;
            if constexpr (R::kVectorStep) {
                // first stage of argmax/argmin: the best value and its row, counted from the slab's
                // first row in 32 bits (the launcher refuses longer slabs), stay in registers; the
                // rows come in increasing order, so only a strictly better value replaces the best
                using V = typename R::Val;
                V best[VEC];
                int brow[VEC];                       // -1: nothing seen yet
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    best[k] = V{};
                    brow[k] = -1;
                }
                int rel = ty;
                for (; r + int64_t(UNROLL - 1) * ROWS < r_end; r += int64_t(UNROLL) * ROWS, rel += UNROLL * ROWS) {
                    vec_t<In, VEC> x[UNROLL];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        const int64_t rr = r + int64_t(u) * ROWS;
                        int64_t off, unused;
                        if (simple) off = rr * rs;
                        else red_offsets(red, rr, off, unused);
                        x[u] = load_vec<vec_t<In, VEC>>(base + off);
                    }
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                        for (int k = 0; k < VEC; ++k) {
                            const V xv = R::value(x[u].v[k]);
                            const bool wins = (brow[k] < 0) | R::beats(xv, best[k]);
                            best[k] = wins ? xv : best[k];
                            brow[k] = wins ? rel + u * ROWS : brow[k];
                        }
                }
                for (; r < r_end; r += ROWS, rel += ROWS) {
                    int64_t off, unused;
                    if (simple) off = r * rs;
                    else red_offsets(red, r, off, unused);
                    vec_t<In, VEC> x = load_vec<vec_t<In, VEC>>(base + off);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) {
                        const V xv = R::value(x.v[k]);
                        const bool wins = (brow[k] < 0) | R::beats(xv, best[k]);
                        best[k] = wins ? xv : best[k];
                        brow[k] = wins ? rel : brow[k];
                    }
                }
#pragma unroll
                for (int k = 0; k < VEC; ++k)
                    if (brow[k] >= 0) {
                        lanes[k].val = best[k];
                        lanes[k].idx = r_begin + brow[k];
                    }
            }
            else {
                for (; r + int64_t(UNROLL - 1) * ROWS < r_end; r += int64_t(UNROLL) * ROWS) {
                    vec_t<In, VEC> x[UNROLL];
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u) {
                        const int64_t rr = r + int64_t(u) * ROWS;
                        int64_t off, unused;
                        if (simple) off = rr * rs;
                        else red_offsets(red, rr, off, unused);
                        x[u] = load_vec<vec_t<In, VEC>>(base + off);
                    }
#pragma unroll
                    for (int u = 0; u < UNROLL; ++u)
#pragma unroll
                        for (int k = 0; k < VEC; ++k)
                            lanes[k] = R::step(lanes[k], x[u].v[k], r + int64_t(u) * ROWS);
                }
                for (; r < r_end; r += ROWS) {
                    int64_t off, unused;
                    if (simple) off = r * rs;
                    else red_offsets(red, r, off, unused);
                    vec_t<In, VEC> x = load_vec<vec_t<In, VEC>>(base + off);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) lanes[k] = R::step(lanes[k], x.v[k], r);
                }
            }
        }
        if constexpr (ROWS > 1) {
            __syncthreads();
#pragma unroll
            for (int k = 0; k < VEC; ++k) smem[ty][tx][k] = lanes[k];
            __syncthreads();
        }
        if (ty == 0 && active) {
#pragma unroll
            for (int k = 0; k < VEC; ++k) {
                Acc a = lanes[k];
                if constexpr (ROWS > 1) {
                    a = smem[0][tx][k];
#pragma unroll
                    for (int j = 1; j < ROWS; ++j) a = R::combine(a, smem[j][tx][k]);
                }
                if (final_pass) red_store<R>(res, b_dst + col + k, a, true);
                else red_store<R>(res, (slab * nbatch + b) * C + col + k, a, false);
            }
        }
    }
}

// ----------------------------------------------------------------- generic
// Work item = (result element, split); GROUP threads walk the reduction index
// space of the item with a stride of GROUP, computing every offset from the
// collapsed reduction dimensions.
template <class R, int GROUP>
__global__ void __launch_bounds__(kRedThreads)
    reduce_generic_kernel(const typename R::In *arg, void *res, RedMeta iter, RedMeta red,
                          int64_t niter, int64_t nred, int64_t nsplit, int64_t chunk, bool final_pass)
{
    using Acc = typename R::Acc;
    __shared__ Acc smem[8];
    constexpr int GROUPS_PER_BLOCK = kRedThreads / GROUP;
    const int g = threadIdx.x / GROUP;
    const int t = threadIdx.x % GROUP;
    const int64_t nitems = niter * nsplit;
    const int64_t nblock_items = (nitems + GROUPS_PER_BLOCK - 1) / GROUPS_PER_BLOCK;
    for (int64_t bi = blockIdx.x; bi < nblock_items; bi += gridDim.x) {
        const int64_t item = bi * GROUPS_PER_BLOCK + g;
        const bool active = item < nitems;
        Acc acc = R::identity();
        int64_t o_src = 0, o_dst = 0;
        if (active) {
            const int64_t out_i = item / nsplit;
            const int64_t split = item - out_i * nsplit;
            red_offsets(iter, out_i, o_src, o_dst);
            const int64_t begin = split * chunk;
            int64_t end = begin + chunk;
            if (end > nred) end = nred;
            for (int64_t e = begin + t; e < end; e += GROUP) {
                int64_t off, unused;
                red_offsets(red, e, off, unused);
                acc = R::step(acc, arg[o_src + off], e);
            }
        }
        acc = group_reduce<R, GROUP>(acc, smem);
        if (active && t == 0) {
            if (final_pass) red_store<R>(res, o_dst, acc, true);
            else red_store<R>(res, item, acc, false);
        }
    }
}

}  // namespace dpb
