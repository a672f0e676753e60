// Accumulation (prefix scan) along one axis for any operator R of reduce_ops.cuh whose
// merge is associative: cumulative sum, product and logsumexp.
//
// Replaces the reference's accumulators (include/kernels/accumulators.hpp: the blocked
// inclusive_scan_base_step / update chain behind _cumsum_over_axis, _cumprod_over_axis and
// _cumlogsumexp_over_axis).  Two kernel shapes:
//   scan_rows   a block walks one row (or one segment of a row) chunk by chunk, carrying
//               the running value: thread-local scan of ITEMS elements, warp scan of the
//               thread totals by shuffles, 8 warp totals through shared memory.  With many
//               rows every row is one block and the data is read once and written once.
//               A few long rows are cut into segments: a first launch of the same kernel
//               only totals the segments, a tiny launch turns the totals into carry-ins,
//               and the main launch scans every segment from its carry-in.  No block ever
//               waits for another block.
//   scan_cols   the scanned axis is strided and the innermost other dimension is
//               unit-stride (C-contiguous, axis 0): a thread owns a column and walks down
//               the rows, so a warp reads and writes 32 adjacent elements per step.
// The partition depends on the sizes only, so results do not change from run to run.
#pragma once

#include "reduce_kernels.cuh"

namespace dpb {

constexpr int kScanThreads = 256;
// column scans use small blocks: all of them are resident at once for the sizes that take this
// path, and many small blocks spread evenly over the SMs where a few large ones would not
constexpr int kScanColThreads = 64;

template <class T> DPB_D T shfl_idx_any(const T &v, int src_lane)
{
    constexpr int W = (sizeof(T) + 3) / 4;
    uint32_t w[W];
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = 0;
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_sync(0xffffffffu, w[i], src_lane);
    T out;
    memcpy(&out, w, sizeof(T));
    return out;
}

template <class T> DPB_D T shfl_up_any(const T &v, int delta)
{
    constexpr int W = (sizeof(T) + 3) / 4;
    uint32_t w[W];
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = 0;
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_up_sync(0xffffffffu, w[i], delta);
    T out;
    memcpy(&out, w, sizeof(T));
    return out;
}

// Work item = (row, segment).  `iter` gives the row's offsets in src and dst; the scanned
// axis has strides s_src / s_dst; segment s covers [s*seg_len, min(L, (s+1)*seg_len)).
// TOTALS_ONLY: nothing is stored but the merged value of the segment (into `totals`).
// `carry_in` (may be null) holds the value every element of the item starts from.
// dst_shift = 1 writes result i to position i+1 (the caller has put the identity at 0).
// UNIT: both strides of the scanned axis are 1.  VEC (needs UNIT): every row start and every
// segment start is aligned for whole-thread accesses (ITEMS elements, in pieces of 16 bytes).
template <class R, int ITEMS, bool UNIT, bool VEC, bool TOTALS_ONLY>
__global__ void __launch_bounds__(kScanThreads)
    scan_rows_kernel(const typename R::In *src, typename R::Out *dst, RedMeta iter, int64_t nrows, int64_t L,
                     int64_t s_src, int64_t s_dst, int64_t nseg, int64_t seg_len,
                     const typename R::Acc *carry_in, typename R::Acc *totals, int64_t dst_shift)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    using Out = typename R::Out;
    __shared__ Acc warp_tot[kScanThreads / 32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t nitems = nrows * nseg;
    for (int64_t item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int64_t row = item / nseg;
        const int64_t seg = item - row * nseg;
        int64_t o_src, o_dst;
        red_offsets(iter, row, o_src, o_dst);
        const int64_t begin = seg * seg_len;
        int64_t end = begin + seg_len;
        if (end > L) end = L;
        const In *p = src + o_src;
        Out *q = dst + o_dst + dst_shift * s_dst;
        Acc carry = carry_in ? carry_in[item] : R::identity();
        // the thread's ITEMS raw elements of the chunk that starts at `base` (elements past the
        // end are left unset and masked when they are used)
        auto fetch = [&](int64_t base, In(&raw)[ITEMS]) {
            const int64_t i0 = base + int64_t(tid) * ITEMS;
            if (VEC && i0 + ITEMS <= end) {
                constexpr int IV = (16 / sizeof(In)) < ITEMS ? (16 / sizeof(In)) : ITEMS;  // per access
#pragma unroll
                for (int g = 0; g < ITEMS; g += IV) {
                    const vec_t<In, IV> x = load_vec<vec_t<In, IV>>(p + i0 + g);
#pragma unroll
                    for (int j = 0; j < IV; ++j) raw[g + j] = x.v[j];
                }
            }
            else {
#pragma unroll
                for (int i = 0; i < ITEMS; ++i) {
                    const int64_t e = i0 + i;
                    if (e < end) raw[i] = UNIT ? p[e] : p[e * s_src];
                }
            }
        };
        constexpr int64_t kChunk = int64_t(kScanThreads) * ITEMS;
        In raw[ITEMS];
        if (begin < end) fetch(begin, raw);
        for (int64_t base = begin; base < end; base += kChunk) {
            const int64_t i0 = base + int64_t(tid) * ITEMS;
            const bool whole = i0 + ITEMS <= end;
            Acc v[ITEMS];
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) v[i] = (i0 + i < end) ? R::load(raw[i], i0 + i) : R::identity();
            // the next chunk's loads are in flight while this one is scanned and stored
            if (base + kChunk < end) fetch(base + kChunk, raw);
#pragma unroll
            for (int i = 1; i < ITEMS; ++i) v[i] = R::combine(v[i - 1], v[i]);
            // inclusive scan of the thread totals inside the warp
            Acc incl = v[ITEMS - 1];
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const Acc up = shfl_up_any(incl, d);
                if (lane >= d) incl = R::combine(up, incl);
            }
            if (lane == 31) warp_tot[warp] = incl;
            __syncthreads();
            Acc before = carry;   // everything before this warp, in order
            Acc chunk_total = R::identity();
#pragma unroll
            for (int w = 0; w < kScanThreads / 32; ++w) {
                const Acc t = warp_tot[w];
                if (w < warp) before = R::combine(before, t);
                chunk_total = R::combine(chunk_total, t);
            }
            if constexpr (!TOTALS_ONLY) {
                Acc excl = shfl_up_any(incl, 1);
                Acc prefix = lane == 0 ? before : R::combine(before, excl);
                if (VEC && whole) {
                    constexpr int OV = (16 / sizeof(Out)) < ITEMS ? (16 / sizeof(Out)) : ITEMS;
#pragma unroll
                    for (int g = 0; g < ITEMS; g += OV) {
                        vec_t<Out, OV> r;
#pragma unroll
                        for (int j = 0; j < OV; ++j) r.v[j] = R::finish(R::combine(prefix, v[g + j]));
                        store_vec(q + i0 + g, r);
                    }
                }
                else {
#pragma unroll
                    for (int i = 0; i < ITEMS; ++i) {
                        const int64_t e = i0 + i;
                        if (e < end) {
                            const Out r = R::finish(R::combine(prefix, v[i]));
                            if (UNIT) q[e] = r;
                            else q[e * s_dst] = r;
                        }
                    }
                }
            }
            carry = R::combine(carry, chunk_total);
            __syncthreads();  // warp_tot is rewritten by the next chunk
        }
        if constexpr (TOTALS_ONLY) {
            if (tid == 0) totals[item] = carry;
        }
    }
}

// Exclusive scan of the nseg segment totals of every row, in place: totals[row][s] becomes
// the merged value of segments 0..s-1.  One warp per row; nseg is at most a few thousand.
template <class R>
__global__ void __launch_bounds__(kScanThreads)
    scan_totals_kernel(typename R::Acc *totals, int64_t nrows, int64_t nseg)
{
    using Acc = typename R::Acc;
    const int lane = threadIdx.x & 31;
    const int64_t row = int64_t(blockIdx.x) * (kScanThreads / 32) + (threadIdx.x >> 5);
    if (row >= nrows) return;
    Acc *t = totals + row * nseg;
    Acc carry = R::identity();
    for (int64_t base = 0; base < nseg; base += 32) {
        const int64_t i = base + lane;
        const Acc mine = i < nseg ? t[i] : R::identity();
        Acc incl = mine;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const Acc up = shfl_up_any(incl, d);
            if (lane >= d) incl = R::combine(up, incl);
        }
        const Acc excl = shfl_up_any(incl, 1);
        if (i < nseg) t[i] = lane == 0 ? carry : R::combine(carry, excl);
        carry = R::combine(carry, shfl_idx_any(incl, 31));
    }
}

// `cols` columns are unit-stride in src and dst; a thread owns one column of one batch entry
// and walks the L rows (stride r_src / r_dst) with 8 to 32 loads in flight.
template <class R>
__global__ void __launch_bounds__(kScanColThreads)
    scan_cols_kernel(const typename R::In *src, typename R::Out *dst, RedMeta batch, int64_t nbatch,
                     int64_t cols, int64_t L, int64_t r_src, int64_t r_dst, int64_t dst_shift)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    const int64_t colblocks = (cols + kScanColThreads - 1) / kScanColThreads;
    const int64_t nwork = nbatch * colblocks;
    for (int64_t w = blockIdx.x; w < nwork; w += gridDim.x) {
        const int64_t b = w / colblocks;
        const int64_t c = (w - b * colblocks) * kScanColThreads + threadIdx.x;
        if (c >= cols) continue;
        int64_t o_src, o_dst;
        red_offsets(batch, b, o_src, o_dst);
        const In *p = src + o_src + c;
        typename R::Out *q = dst + o_dst + c + dst_shift * r_dst;
        Acc acc = R::identity();
        int64_t r = 0;
        // loads in flight per thread: 128 bytes' worth
        constexpr int U = sizeof(In) >= 16 ? 8 : (128 / sizeof(In) > 32 ? 32 : (128 / sizeof(In) < 8 ? 8 : 128 / sizeof(In)));
        for (; r + U <= L; r += U) {
            In x[U];
#pragma unroll
            for (int u = 0; u < U; ++u) x[u] = p[(r + u) * r_src];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                acc = R::combine(acc, R::load(x[u], r + u));
                q[(r + u) * r_dst] = R::finish(acc);
            }
        }
        for (; r < L; ++r) {
            acc = R::combine(acc, R::load(p[r * r_src], r));
            q[r * r_dst] = R::finish(acc);
        }
    }
}

}  // namespace dpb
