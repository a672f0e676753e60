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

// ------------------------------------------------------------ single pass over long rows
// A few long rows in ONE pass over the data (read once, written once): the row is cut into tiles of
// kScanThreads * ITEMS elements, one block per tile.  A block scans its tile in registers,
// publishes the tile's total, obtains the merged value of everything before its tile from what
// the earlier tiles have published, and stores.  A block only ever waits for blocks with smaller
// indices, which started before it and are running or finished.
//
// What a tile merges, and in which order, depends on its index alone (results do not change
// from run to run): the totals form a tree of radix 32.  Level 0 holds the tile totals T[i];
// an entry g of level k+1 is the warp-fold (the inclusive shuffle scan's last lane) of entries
// 32g .. 32g+31 of level k, published by the tile that closes the group.  With the tile index
// written in base 32 as (a3 a2 a1 a0), the value before the tile is
//     fold(level3[.. a3)) + fold(level2[.. a2 of its group)) + fold(level1[..a1)) + fold(T[..a0))
// -- at most 31 entries per level, loaded by one warp.
//
// Every wait is bounded (max_polls probes with a short sleep between them).  A tile whose wait runs
// out stores nothing, leaves its `done` word at 0 and raises `*error`; two repair launches that
// follow on the stream (and return at once when `*error` is 0) then build the upper levels from
// the tile totals -- every tile publishes its total before it waits for anything -- and redo the
// tiles that are not done, with the same folds, so the bits are those of the undisturbed run.
//
// Measured on B200 (2^28 float32 in one row): 0.94 ms against 0.58 ms for the three launches of
// scan_rows above, although those read the data twice.  A tile holds its block for the load plus
// two to three round trips to L2 (its neighbours publish when it does, so the first probe rarely
// finds them), about 8 us, and the registers of the resident blocks hold 64 KB per SM -- a third of
// what HBM needs in flight at that latency.  Splitting the tile into a publishing and a finishing
// phase some steps apart (second read from L2) reached 0.72 ms, two tiles' loads in flight per block
// 0.95 ms (fewer resident blocks).  So the path is off unless the "scan_lookback_polls" switch asks
// for it; the tests run both.
constexpr int kLookbackLevels = 4;          // 32^4 tiles per row at most

struct LookbackLayout {
    int levels;                             // levels in use (1: a row of at most 32 tiles)
    int64_t n[kLookbackLevels];             // entries per level and row
    int64_t off[kLookbackLevels];           // start of the level within a row's block of entries
    int64_t per_row;                        // entries per row
};

template <class T> DPB_D T load_cg(const T *p)
{
    // past L1, which is not coherent between SMs
    if constexpr (sizeof(T) == 16) {
        const uint4 w = __ldcg(reinterpret_cast<const uint4 *>(p));
        T out;
        memcpy(&out, &w, 16);
        return out;
    }
    else if constexpr (sizeof(T) == 8) {
        const unsigned long long w = __ldcg(reinterpret_cast<const unsigned long long *>(p));
        T out;
        memcpy(&out, &w, 8);
        return out;
    }
    else if constexpr (sizeof(T) == 4) {
        const unsigned w = __ldcg(reinterpret_cast<const unsigned *>(p));
        T out;
        memcpy(&out, &w, 4);
        return out;
    }
    else if constexpr (sizeof(T) == 2) {
        const unsigned short w = __ldcg(reinterpret_cast<const unsigned short *>(p));
        T out;
        memcpy(&out, &w, 2);
        return out;
    }
    else {
        static_assert(sizeof(T) == 1, "accumulator size");
        const unsigned char w = __ldcg(reinterpret_cast<const unsigned char *>(p));
        T out;
        memcpy(&out, &w, 1);
        return out;
    }
}

DPB_D unsigned flag_load(const unsigned *p)
{
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

DPB_D void flag_store(unsigned *p, unsigned v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// How an entry (a tile total or a group's fold) travels between blocks.  A 4-byte value shares one
// 8-byte word with its flag: one store publishes both and one load probes and fetches.  Larger
// values sit beside a separate flag word: value, release-store of the flag; probe of the flag,
// fence, load of the value past L1.
template <class Acc> struct LookbackEntries {
    static constexpr bool kPacked = sizeof(Acc) == 4;
    static constexpr size_t kValueBytes = kPacked ? 8 : sizeof(Acc);
    void *vals;          // kPacked: 8-byte words (value | flag << 32); else Acc
    unsigned *flags;     // unused when kPacked

    DPB_D void publish(int64_t e, const Acc &v) const
    {
        if constexpr (kPacked) {
            unsigned bits;
            memcpy(&bits, &v, 4);
            const unsigned long long w = (1ull << 32) | bits;
            asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(static_cast<unsigned long long *>(vals) + e), "l"(w)
                         : "memory");
        }
        else {
            static_cast<Acc *>(vals)[e] = v;
            flag_store(flags + e, 1u);
        }
    }
    // one probe; kPacked: the value comes with it
    DPB_D bool probe(int64_t e, Acc &v) const
    {
        if constexpr (kPacked) {
            unsigned long long w;
            asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];"
                         : "=l"(w)
                         : "l"(static_cast<const unsigned long long *>(vals) + e)
                         : "memory");
            if ((w >> 32) == 0) return false;
            const unsigned bits = static_cast<unsigned>(w);
            memcpy(&v, &bits, 4);
            return true;
        }
        else {
            return flag_load(flags + e) != 0;
        }
    }
    // the value of an entry whose flag has been seen (after a fence) or that is known to be there
    DPB_D Acc fetch(int64_t e) const
    {
        if constexpr (kPacked) {
            const unsigned long long w = __ldcg(static_cast<const unsigned long long *>(vals) + e);
            const unsigned bits = static_cast<unsigned>(w);
            Acc v;
            memcpy(&v, &bits, 4);
            return v;
        }
        else {
            return load_cg(static_cast<const Acc *>(vals) + e);
        }
    }
};

// the warp-fold: ordered merge of the 32 lanes' values, the same tree wherever it is used
template <class R> DPB_D typename R::Acc warp_fold(typename R::Acc x, int lane)
{
    using Acc = typename R::Acc;
    Acc incl = x;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const Acc up = shfl_up_any(incl, d);
        if (lane >= d) incl = R::combine(up, incl);
    }
    return shfl_idx_any(incl, 31);
}

// One tile.  REPAIR = false: the single pass (entries are waited for and published).  REPAIR = true:
// every entry is there already, nothing is waited for or published.
template <class R, int ITEMS, bool VEC, bool REPAIR>
DPB_D void lookback_tile(int64_t t, const typename R::In *src, typename R::Out *dst, const RedMeta &iter, int64_t L,
                         int64_t ntiles, const LookbackLayout &lay, LookbackEntries<typename R::Acc> ent,
                         unsigned *done, unsigned *error, int max_polls, int64_t dst_shift)
{
    using In = typename R::In;
    using Acc = typename R::Acc;
    using Out = typename R::Out;
    __shared__ Acc warp_tot[kScanThreads / 32];
    __shared__ Acc s_prefix;
    __shared__ int s_fail;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t row = t / ntiles, tile = t - row * ntiles;
    int64_t o_src, o_dst;
    red_offsets(iter, row, o_src, o_dst);
    constexpr int64_t kChunk = int64_t(kScanThreads) * ITEMS;
    const int64_t begin = tile * kChunk;
    const int64_t end = begin + kChunk < L ? begin + kChunk : L;
    const In *p = src + o_src;
    Out *q = dst + o_dst + dst_shift;
    const int64_t i0 = begin + int64_t(tid) * ITEMS;
    const bool whole = i0 + ITEMS <= end;

    // ---- the tile, scanned in registers
    Acc v[ITEMS];
    if (VEC && whole) {
        constexpr int IV = (16 / sizeof(In)) < ITEMS ? (16 / sizeof(In)) : ITEMS;
#pragma unroll
        for (int g = 0; g < ITEMS; g += IV) {
            const vec_t<In, IV> x = load_vec<vec_t<In, IV>>(p + i0 + g);
#pragma unroll
            for (int j = 0; j < IV; ++j) v[g + j] = R::load(x.v[j], i0 + g + j);
        }
    }
    else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) v[i] = (i0 + i < end) ? R::load(p[i0 + i], i0 + i) : R::identity();
    }
#pragma unroll
    for (int i = 1; i < ITEMS; ++i) v[i] = R::combine(v[i - 1], v[i]);
    Acc incl = v[ITEMS - 1];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const Acc up = shfl_up_any(incl, d);
        if (lane >= d) incl = R::combine(up, incl);
    }
    __syncthreads();              // the previous tile of this block (repair) is done with the shared words
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    Acc before = R::identity();   // the warps of this tile before mine, in order
    Acc tile_total = R::identity();
#pragma unroll
    for (int w = 0; w < kScanThreads / 32; ++w) {
        const Acc tw = warp_tot[w];
        if (w < warp) before = R::combine(before, tw);
        tile_total = R::combine(tile_total, tw);
    }

    // ---- what comes before the tile
    const int64_t rbase = row * lay.per_row;      // the row's block of entries
    if (warp == 0) {
        constexpr unsigned kAll = 0xffffffffu;
        constexpr bool kPacked = LookbackEntries<Acc>::kPacked;
        if constexpr (!REPAIR) {
            if (lane == 0) ent.publish(rbase + lay.off[0] + tile, tile_total);
        }
        // Every lane looks after one predecessor per level; all levels are probed together, so the
        // wait is the slowest entry's, not the sum over the levels.
        int digit[kLookbackLevels];
        int64_t entry[kLookbackLevels];       // this lane's predecessor at the level (if lane < digit)
        Acc x[kLookbackLevels];               // its value
        {
            int64_t idx = tile;
#pragma unroll
            for (int lev = 0; lev < kLookbackLevels; ++lev) {
                digit[lev] = lev < lay.levels ? static_cast<int>(idx & 31) : 0;
                entry[lev] = rbase + lay.off[lev] + (idx - digit[lev]) + lane;
                x[lev] = R::identity();
                idx >>= 5;
            }
        }
        bool fail = false;
        if constexpr (!REPAIR) {
            unsigned pending = 0;
#pragma unroll
            for (int lev = 0; lev < kLookbackLevels; ++lev)
                if (lane < digit[lev]) pending |= 1u << lev;
            // The last member of a full group publishes the group's entry one level up -- as soon
            // as that level's 31 predecessors are there, whatever the other levels still wait for
            // (the tiles of the next group wait for this entry).
            int closing = 0;                  // level whose group this tile closes next
            Acc mine = tile_total;            // the tile's own entry at that level
            int polls = 0;
            while (true) {
#pragma unroll
                for (int lev = 0; lev < kLookbackLevels; ++lev)
                    if ((pending >> lev) & 1u)
                        if (ent.probe(entry[lev], x[lev])) pending &= ~(1u << lev);
#pragma unroll
                for (int lev = 0; lev + 1 < kLookbackLevels; ++lev) {
                    if (closing == lev) {
                        if (lev + 1 >= lay.levels || digit[lev] != 31) closing = kLookbackLevels;   // none left
                        else if (!__any_sync(kAll, (pending >> lev) & 1u)) {
                            Acc y;
                            if constexpr (kPacked) y = lane < 31 ? x[lev] : mine;
                            else {
                                __threadfence();          // entries are read after their flags
                                y = lane < 31 ? ent.fetch(entry[lev]) : mine;
                            }
                            mine = warp_fold<R>(y, lane);
                            if (lane == 0) ent.publish(rbase + lay.off[lev + 1] + (tile >> (5 * (lev + 1))), mine);
                            closing = lev + 1;
                        }
                    }
                }
                if (!__any_sync(kAll, pending != 0)) break;
                const bool stop = polls >= max_polls || ((polls & 63) == 63 && flag_load(error) != 0);
                if (__any_sync(kAll, stop)) {
                    fail = true;
                    break;
                }
                ++polls;
                if (polls > 64) __nanosleep(100);
            }
            if constexpr (!kPacked) __threadfence();      // entries are read after their flags
        }
        if (REPAIR || !kPacked) {
#pragma unroll
            for (int lev = 0; lev < kLookbackLevels; ++lev)
                if (lane < digit[lev] && !fail) x[lev] = ent.fetch(entry[lev]);
        }
        Acc prefix = R::identity();
#pragma unroll
        for (int lev = kLookbackLevels - 1; lev >= 0; --lev)
            if (lev < lay.levels) prefix = R::combine(prefix, warp_fold<R>(lane < digit[lev] ? x[lev] : R::identity(), lane));
        if (lane == 0) {
            s_prefix = prefix;
            s_fail = fail ? 1 : 0;
        }
    }
    __syncthreads();
    if (s_fail) {
        if (tid == 0) atomicExch(error, 1u);
        return;
    }
    // ---- store
    const Acc excl = shfl_up_any(incl, 1);
    Acc prefix = R::combine(s_prefix, before);
    if (lane != 0) prefix = R::combine(prefix, excl);
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
        for (int i = 0; i < ITEMS; ++i)
            if (i0 + i < end) q[i0 + i] = R::finish(R::combine(prefix, v[i]));
    }
    if constexpr (!REPAIR) {
        if (tid == 0) done[t] = 1u;
    }
}

// The single pass: one tile per block, in the order of the block index.  (Blocks of a
// one-dimensional grid start in that order on this hardware; the design does not depend on it --
// a tile whose predecessors have not started would run out of probes and be redone by the repair
// launches -- it only saves every tile a round trip to a ticket counter.)
template <class R, int ITEMS, bool VEC>
__global__ void __launch_bounds__(kScanThreads)
    scan_lookback_kernel(const typename R::In *src, typename R::Out *dst, RedMeta iter, int64_t L, int64_t ntiles,
                         LookbackLayout lay, LookbackEntries<typename R::Acc> ent, unsigned *done, unsigned *error,
                         int max_polls, int64_t dst_shift)
{
    lookback_tile<R, ITEMS, VEC, false>(blockIdx.x, src, dst, iter, L, ntiles, lay, ent, done, error, max_polls,
                                        dst_shift);
}

// After a single pass that raised `*error` (and after scan_lookback_levels_kernel): the tiles whose
// `done` word is 0.  A small grid walks the tiles; it returns at once when there was no error.
template <class R, int ITEMS, bool VEC>
__global__ void __launch_bounds__(kScanThreads)
    scan_lookback_repair_kernel(const typename R::In *src, typename R::Out *dst, RedMeta iter, int64_t nrows,
                                int64_t L, int64_t ntiles, LookbackLayout lay, LookbackEntries<typename R::Acc> ent,
                                unsigned *done, unsigned *error, int64_t dst_shift)
{
    if (flag_load(error) == 0) return;
    for (int64_t t = blockIdx.x; t < nrows * ntiles; t += gridDim.x) {
        if (flag_load(done + t) != 0) continue;
        lookback_tile<R, ITEMS, VEC, true>(t, src, dst, iter, L, ntiles, lay, ent, done, error, 0, dst_shift);
    }
}

// After a single pass that raised `*error`: levels 1.. of every row rebuilt from the tile totals
// with the folds of the single pass.  One block; the levels follow one another.
template <class R>
__global__ void __launch_bounds__(1024)
    scan_lookback_levels_kernel(LookbackEntries<typename R::Acc> ent, LookbackLayout lay, int64_t nrows,
                                const unsigned *error)
{
    using Acc = typename R::Acc;
    if (flag_load(error) == 0) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int lev = 1; lev < lay.levels; ++lev) {
        for (int64_t row = 0; row < nrows; ++row) {
            const int64_t rbase = row * lay.per_row;
            for (int64_t g = warp; g < lay.n[lev]; g += nwarps) {
                const int64_t e = g * 32 + lane;
                const Acc x = e < lay.n[lev - 1] ? ent.fetch(rbase + lay.off[lev - 1] + e) : R::identity();
                const Acc f = warp_fold<R>(x, lane);
                if (lane == 0) ent.publish(rbase + lay.off[lev] + g, f);
            }
        }
        __threadfence();
        __syncthreads();
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
